// Linear attention with a fixed decay per head, as a recurrence over a per-sequence state:
//
//   S_t = decay_h * S_{t-1} + k_t v_t^T          (S: [d, dv] float32 per sequence and head)
//   o_t = S_t^T q_t
//
// q, k (heads x d) and v (heads x dv) are columns of the packed float32 projection [T, ld]; on their
// way in they may pass an activation (silu), a rotate-half rotation of their first `rot` channels by
// the token's position (q and k only; table float32 [positions, rot / 2, 2]) and a constant factor
// on k, in that order.  The state lives in the cache's per-sequence storage, [slots, heads, d, dv]
// float32; a step loads it, runs its tokens in order and stores it, so prompts, portions of
// prompts and single tokens are the same code and carry the same bits from step to step.
//
// decay_scan_kernel: one block per (sequence, head).  The state sits in shared memory for the
// step; the step's tokens come in tiles of DS_TILE, prepared (activation, rotation, factor) by all
// threads; then the tokens of the tile run one after the other: thread (r, j) owns rows r, r + R, ..
// of column j, updates them and adds up its part of o_t[j]; the R parts are added in a fixed order.
//
// decay_chunk_kernel: the same recurrence for prompts in chunks of DC_C tokens on the tensor cores'
// float32-accumulating warp MMAs is not what this file does: everything here is float32 FMA, so that
// the float32 mode and the bfloat16 mode share one implementation of the recurrence, which the
// design asks to be float32 in both.
//
// group_norm_gate_kernel: what follows the recurrence in such mixers: an RMS norm over groups of the
// concatenated heads (one group = all heads together, with a weight; or one group per head, without),
// times an activation of a gate projection (sigmoid or silu), rounded once to the activation dtype.
#include "common.cuh"

#define DS_TILE 16
#define DS_THREADS 256

struct DecayScanArgs {
    const float* x;
    int ld, q_off, k_off, v_off;
    int nh, d, dv;
    int qk_act, v_act;              // 0: none, 1: silu
    const float* cos_sin;
    int rot, n_pos;
    float k_scale;
    const float* decay;             // [nh]
    float* state;                   // [slots, nh, d, dv]
    const int *slots, *cu_q, *token_pos;
    float* out;                     // [T, nh * dv]
    int* err;
};

__device__ __forceinline__ float act_of(float v, int act) {
    if (act == 1) return v / (1.0f + expf(-v));
    if (act == 2) return 1.0f / (1.0f + expf(-v));
    return v;
}

__global__ void __launch_bounds__(DS_THREADS) decay_scan_kernel(DecayScanArgs a) {
    pdl_grid_sync();
    extern __shared__ float sm[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int d = a.d, dv = a.dv;
    float* S = sm;                          // [d][dv]
    float* qt = S + (size_t)d * dv;         // [DS_TILE][d]
    float* kt = qt + DS_TILE * d;           // [DS_TILE][d]
    float* vt = kt + DS_TILE * d;           // [DS_TILE][dv]
    float* red = vt + DS_TILE * dv;         // [R][dv]
    // columns per pass and row groups: a function of dv alone
    const int J = dv < DS_THREADS ? ((dv + 31) & ~31) : DS_THREADS;
    const int R = DS_THREADS / J;
    const int r = threadIdx.x / J, jj = threadIdx.x % J;
    const float dec = a.decay[h];
    float* Sg = a.state + ((size_t)a.slots[b] * a.nh + h) * (size_t)d * dv;
    for (int i = threadIdx.x; i < d * dv; i += DS_THREADS) S[i] = Sg[i];
    const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
    const int half = a.rot >> 1;
    for (int tb = t0; tb < t1; tb += DS_TILE) {
        const int n = t1 - tb < DS_TILE ? t1 - tb : DS_TILE;
        __syncthreads();        // the previous tile has been used (and S is loaded)
        for (int i = threadIdx.x; i < n * d; i += DS_THREADS) {
            const int tt = i / d, c = i - tt * d;
            const float* row = a.x + (size_t)(tb + tt) * a.ld;
            float q = act_of(row[a.q_off + h * d + c], a.qk_act);
            float k = act_of(row[a.k_off + h * d + c], a.qk_act);
            if (c < a.rot) {
                int p = a.token_pos[tb + tt];
                if (p < 0 || p >= a.n_pos) {
                    atomicExch(a.err, 3);
                    p = 0;
                }
                const bool first = c < half;
                const int j = first ? c : c - half, partner = first ? c + half : c - half;
                const float cs = a.cos_sin[((size_t)p * half + j) * 2], sn = a.cos_sin[((size_t)p * half + j) * 2 + 1];
                const float q2 = act_of(row[a.q_off + h * d + partner], a.qk_act);
                const float k2 = act_of(row[a.k_off + h * d + partner], a.qk_act);
                q = first ? q * cs - q2 * sn : q * cs + q2 * sn;
                k = first ? k * cs - k2 * sn : k * cs + k2 * sn;
            }
            qt[i] = q;
            kt[i] = k * a.k_scale;
        }
        for (int i = threadIdx.x; i < n * dv; i += DS_THREADS) {
            const int tt = i / dv, c = i - tt * dv;
            vt[i] = act_of(a.x[(size_t)(tb + tt) * a.ld + a.v_off + h * dv + c], a.v_act);
        }
        __syncthreads();
        for (int tt = 0; tt < n; tt++) {
            const float* q = qt + tt * d;
            const float* k = kt + tt * d;
            const float* v = vt + tt * dv;
            for (int j = jj; j < dv; j += J) {
                const float vj = v[j];
                float part = 0.f;
                if (r < R)
                    for (int i = r; i < d; i += R) {
                        const float s = dec * S[i * dv + j] + k[i] * vj;
                        S[i * dv + j] = s;
                        part = fmaf(s, q[i], part);
                    }
                if (r < R) red[r * dv + j] = part;
            }
            __syncthreads();
            for (int j = threadIdx.x; j < dv; j += DS_THREADS) {
                float o = 0.f;
                for (int rr = 0; rr < R; rr++) o += red[rr * dv + j];
                a.out[(size_t)(tb + tt) * a.nh * dv + (size_t)h * dv + j] = o;
            }
            __syncthreads();
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d * dv; i += DS_THREADS) Sg[i] = S[i];
}

extern "C" long long illm_decay_scan_smem(int d, int dv) {
    const int J = dv < DS_THREADS ? ((dv + 31) & ~31) : DS_THREADS;
    const int R = DS_THREADS / J;
    return ((long long)d * dv + 2LL * DS_TILE * d + (long long)DS_TILE * dv + (long long)R * dv) * (long long)sizeof(float);
}

extern "C" int illm_decay_scan(const float* x, int ld, int q_off, int k_off, int v_off, int nh, int d, int dv, int qk_act, int v_act,
                               const float* cos_sin, int rot, int n_pos, float k_scale, const float* decay, float* state, const int* slots,
                               const int* cu_q, const int* token_pos, float* out, int B, int* err, void* stream) {
    if (B <= 0) return 0;
    if (nh <= 0 || d <= 0 || dv <= 0 || nh > 65535 || rot < 0 || rot > d || (rot & 1) || (rot && !cos_sin) || !x || !state || !out)
        return ILLM_ERR_BAD_ARG;
    const long long smem = illm_decay_scan_smem(d, dv);
    if (smem > 220 * 1024) return ILLM_ERR_BAD_ARG;
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    DecayScanArgs a{x, ld, q_off, k_off, v_off, nh, d, dv, qk_act, v_act, cos_sin, rot, n_pos, k_scale, decay, state, slots, cu_q, token_pos, out, err};
    illm_launch(decay_scan_kernel, dim3(B, nh), dim3(DS_THREADS), (size_t)smem, (cudaStream_t)stream, a);
    return illm_launch_status();
}

// y[t, g, :] = o[t, g, :] / sqrt(mean_g(o^2) + eps) (* w) * act(gate[t, g, :]);  one block per (token, group)
template <typename TA>
__global__ void __launch_bounds__(128)
group_norm_gate_kernel(const float* __restrict__ o, int width, int group, const float* __restrict__ w, float eps,
                       const float* __restrict__ gate, int gate_ld, int gate_act, TA* __restrict__ y) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    const int t = blockIdx.x, g0 = blockIdx.y * group;
    const float* row = o + (size_t)t * width + g0;
    float ss = 0.f;
    for (int c = threadIdx.x; c < group; c += blockDim.x) ss += row[c] * row[c];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)group + eps);
    for (int c = threadIdx.x; c < group; c += blockDim.x) {
        float v = row[c] * inv;
        if (w) v *= w[g0 + c];
        if (gate) v *= act_of(gate[(size_t)t * gate_ld + g0 + c], gate_act);
        y[(size_t)t * width + g0 + c] = from_f32<TA>(v);
    }
}

extern "C" int illm_group_norm_gate(const float* o, int T, int width, int group, const float* w, float eps, const float* gate, int gate_ld,
                                    int gate_act, void* y, int act_dtype, void* stream) {
    if (T <= 0) return 0;
    if (width <= 0 || group <= 0 || width % group || width / group > 65535 || !o || !y) return ILLM_ERR_BAD_ARG;
    dim3 grid(T, width / group);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16)
        illm_launch(group_norm_gate_kernel<bf16>, grid, dim3(128), 0, s, o, width, group, w, eps, gate, gate_ld, gate_act, (bf16*)y);
    else if (act_dtype == ILLM_F32)
        illm_launch(group_norm_gate_kernel<float>, grid, dim3(128), 0, s, o, width, group, w, eps, gate, gate_ld, gate_act, (float*)y);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}
