// The gated delta rule with a decay per head and key channel, over per-sequence state.
//
// Per head, with the state S [d, dv] float32 (zero when a sequence starts), for every token in order:
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// so the read-out sees the token's own write.  Before that, per token (delta_prep_kernel):
//     q, k, v  = silu(conv(projection))     a causal convolution over time per channel, `taps` wide, the last
//                                           tap the token's own, zeros before the sequence's start
//     q, k     = x / sqrt(sum(x^2) + 1e-6) per head;  q also times q_scale
//     beta     = sigmoid(b)                 one per head
//     g        = exp(-exp(A_log_h) * softplus(a + dt_bias))      one per head and key channel
// Query/key head of value head h: h / (heads / kv_heads).  The last taps - 1 rows of the raw q, k, v projections
// are per-sequence state as well ([taps - 1, channels] behind S in a slot's row), renewed by conv_state_kernel
// after the preparation has read them.  Everything here is float32 in both modes of the engine.
//
// delta_scan_kernel: the columns of S never meet, so a block owns (sequence, head, a group of columns); a column's
// d rows are spread over L lanes (L the smallest power of two that leaves a thread at most 32 rows; heads of up to
// 512 key channels) and live in registers for the whole step.  The step's tokens are staged through shared memory in tiles.  The two dot
// products of a token are added over the L lanes by a fixed tree of shuffles, and a token's arithmetic does not
// depend on where the step's cut falls, so prompts, portions and single tokens give the same bits.
#include "common.cuh"

#define DL_THREADS 128
#define DL_ROWS 32
#define DL_TILE 16
#define DL_PREP_TOKENS 4

struct DeltaArgs {
    const float* x;                 // [T, ld] the packed float32 projection
    int T, prep_tokens, ld, q_off, k_off, v_off, b_off;
    const float* a;                 // [T, nh * d] decay projection (before the bias)
    int nh, nkv, d, dv, taps;
    const float *conv_q, *conv_k, *conv_v;      // [channels, taps]
    const float *a_log, *dt_bias;               // [nh], [nh * d]
    float q_scale;
    float* state;                   // [slots, state_elems]: S [nh, dv, d], then the convolution's rows [taps - 1, C]
    long long state_elems;
    const int *slots, *cu_q, *token_pos, *token_seq, *seq_lens;
    float* qkv;                     // out [T, C] prepared q, k, v (C = 2 nkv d + nh dv)
    float* g;                       // out [T, nh * d]
    float* beta;                    // out [T, nh]
    float* out;                     // [T, nh * dv]
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// The convolution of one channel at token t: the taps oldest first, one chain of fused multiply-adds, the same whether a
// row comes from the step or from the state.  KT > 0: the number of taps at compile time; a token that has all its
// earlier rows in the step itself (every token of a prompt but the first few) reads them with fixed offsets.
template <int KT>
__device__ __forceinline__ float conv_channel(const DeltaArgs& p, int t, int i_step, int pos, int c, int col, const float* __restrict__ taps,
                                              const float* __restrict__ conv_state, int C) {
    const int K = KT > 0 ? KT : p.taps;
    const float* xc = p.x + (size_t)t * p.ld + col;
    float y = 0.f;
    if (KT > 0 && i_step >= KT - 1) {
        float in[KT > 0 ? KT : 1], w[KT > 0 ? KT : 1];
#pragma unroll
        for (int j = 0; j < KT; j++) {
            in[j] = __ldg(xc - (ptrdiff_t)j * p.ld);
            w[j] = __ldg(taps + KT - 1 - j);
        }
#pragma unroll
        for (int j = KT - 1; j >= 0; j--) y = fmaf(w[j], in[j], y);
        return y;
    }
    if (KT > 0) {          // the first tokens of a step: rows from the state and from the step, all loads before the chain
        float in[KT > 0 ? KT : 1], w[KT > 0 ? KT : 1];
#pragma unroll
        for (int j = 0; j < KT; j++) {
            in[j] = 0.f;
            w[j] = __ldg(taps + KT - 1 - j);
            if (pos - j >= 0) in[j] = j <= i_step ? __ldg(xc - (ptrdiff_t)j * p.ld) : conv_state[(size_t)(KT - 1 - (j - i_step)) * C + c];
        }
#pragma unroll
        for (int j = KT - 1; j >= 0; j--)
            if (pos - j >= 0) y = fmaf(w[j], in[j], y);
        return y;
    }
    for (int j = K - 1; j >= 0; j--) {
        if (pos - j < 0) continue;
        const float in = j <= i_step ? xc[-(ptrdiff_t)j * p.ld] : conv_state[(size_t)(K - 1 - (j - i_step)) * C + c];
        y = fmaf(taps[K - 1 - j], in, y);
    }
    return y;
}

// silu of a convolved projection: the fast exponential and division (these values may be rounded to bfloat16 anyway)
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// grid (tokens, units), 256 threads.  A unit is a group of query or key heads (convolution, silu, unit vectors; as many
// heads as fit 256 threads, a head of more than 256 channels alone), a piece of 1024 value channels (convolution, silu),
// a piece of 1024 decay channels, or the write strengths of all heads.
__device__ __forceinline__ int delta_heads_per_block(int d) { return d > 256 ? 1 : 256 / ((d + 31) / 32 * 32); }

template <int KT>
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaArgs p) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    __shared__ float warp_ss[8];
    const int unit = blockIdx.y;
    // in a long step a block takes DL_PREP_TOKENS tokens in turn (one in a short step): the look-ups at the start of a token are a chain of dependent loads,
    // which a block of one token would spend most of its life on
#pragma unroll 1
    for (int t = blockIdx.x * p.prep_tokens; t < min(p.T, (int)(blockIdx.x + 1) * p.prep_tokens); t++) {
    __syncthreads();
    const int seq = p.token_seq[t], pos = p.token_pos[t];
    const int i_step = t - p.cu_q[seq];            // the token's place among the step's tokens of its sequence
    const int d = p.d, nq = p.nkv * d, nv = p.nh * p.dv, ng = p.nh * d, C = 2 * nq + nv, K = p.taps;
    const float* conv_state = p.state + (size_t)p.slots[seq] * p.state_elems + (size_t)p.nh * d * p.dv;
    float* dst = p.qkv + (size_t)t * C;
    const int hpb = delta_heads_per_block(d), qk_units = (2 * p.nkv + hpb - 1) / hpb;
    const int v_units = (nv + 1023) / 1024, g_units = (ng + 1023) / 1024;
    if (unit < qk_units && d <= 256) {
        // thread -> (head of the unit, channel); a head's sum of squares: its warps' sums added in order
        const int dth = (d + 31) / 32 * 32, hl = threadIdx.x / dth, i = threadIdx.x % dth;
        const int head = unit * hpb + hl;           // 0 .. nkv - 1 query heads, then the key heads
        const bool live = hl < hpb && head < 2 * p.nkv && i < d;
        const bool is_q = head < p.nkv;
        const int hh = is_q ? head : head - p.nkv;
        float v = 0.f;
        if (live)
            v = silu_fast(conv_channel<KT>(p, t, i_step, pos, head * d + i, (is_q ? p.q_off : p.k_off) + hh * d + i,
                                    (is_q ? p.conv_q : p.conv_k) + ((size_t)hh * d + i) * K, conv_state, C));
        const float ws = warp_sum(v * v);
        if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ws;
        __syncthreads();
        if (live) {
            float ss = 0.f;
            for (int w = hl * (dth / 32); w < (hl + 1) * (dth / 32); w++) ss += warp_ss[w];
            dst[head * d + i] = v * ((1.0f / sqrtf(ss + 1e-6f)) * (is_q ? p.q_scale : 1.0f));
        }
    } else if (unit < qk_units) {
        const bool is_q = unit < p.nkv;
        const int hh = is_q ? unit : unit - p.nkv;
        const float* taps = (is_q ? p.conv_q : p.conv_k) + (size_t)hh * d * K;
        const int c0 = unit * d, col0 = (is_q ? p.q_off : p.k_off) + hh * d;
        float v[2], ss = 0.f;                       // up to 512 channels per head
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int i = threadIdx.x + r * 256;
            v[r] = 0.f;
            if (i < d) {
                v[r] = silu_fast(conv_channel<KT>(p, t, i_step, pos, c0 + i, col0 + i, taps + (size_t)i * K, conv_state, C));
                ss = fmaf(v[r], v[r], ss);
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = (1.0f / sqrtf(ss + 1e-6f)) * (is_q ? p.q_scale : 1.0f);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int i = threadIdx.x + r * 256;
            if (i < d) dst[c0 + i] = v[r] * inv;
        }
    } else if (unit < qk_units + v_units) {
        float y[4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int c = (unit - qk_units) * 1024 + r * 256 + threadIdx.x;
            y[r] = c < nv ? conv_channel<KT>(p, t, i_step, pos, 2 * nq + c, p.v_off + c, p.conv_v + (size_t)c * K, conv_state, C) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int c = (unit - qk_units) * 1024 + r * 256 + threadIdx.x;
            if (c < nv) dst[2 * nq + c] = silu_fast(y[r]);
        }
    } else if (unit < qk_units + v_units + g_units) {
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int c = (unit - qk_units - v_units) * 1024 + r * 256 + threadIdx.x;
            if (c < ng) {
                const float z = p.a[(size_t)t * ng + c] + p.dt_bias[c];
                const float sp = z > 20.f ? z : log1pf(expf(z));
                p.g[(size_t)t * ng + c] = expf(-expf(p.a_log[c / d]) * sp);
            }
        }
    } else {
        for (int h = threadIdx.x; h < p.nh; h += blockDim.x) p.beta[(size_t)t * p.nh + h] = 1.0f / (1.0f + expf(-p.x[(size_t)t * p.ld + p.b_off + h]));
    }
    }
}

// The convolution's rows after the step: the raw projections of the sequence's last taps - 1 positions (zeros for
// positions before its start).  A thread owns a channel and goes through the rows in ascending order, so that a
// row kept from before the step is read before it is overwritten.
__global__ void conv_state_kernel(DeltaArgs p) {
    pdl_grid_sync();
    const int b = blockIdx.y;
    const int nq = p.nkv * p.d, nv = p.nh * p.dv, C = 2 * nq + nv, K = p.taps;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int col = c < nq ? p.q_off + c : c < 2 * nq ? p.k_off + c - nq : p.v_off + c - 2 * nq;
    const int first = p.cu_q[b], n = p.cu_q[b + 1] - first;
    const int len = p.seq_lens[b], past = len - n;
    float* cs = p.state + (size_t)p.slots[b] * p.state_elems + (size_t)p.nh * p.d * p.dv;
    for (int r = 0; r < K - 1; r++) {
        const int pos = len - (K - 1) + r;
        float v = 0.f;
        if (pos >= past) v = p.x[(size_t)(first + pos - past) * p.ld + col];
        else if (pos >= 0) v = cs[(size_t)(r + n) * C + c];
        cs[(size_t)r * C + c] = v;
    }
}

// grid (column groups, heads, sequences); L lanes per column, DL_THREADS / L columns per block.  A thread's 32 rows are
// the quads 4 (l + L r) .. + 3 for r = 0..7, so that its q, k and g come as 16-byte reads of shared memory that the
// lanes of a column make side by side; rows beyond d are padding (k = q = 0, so their state stays 0).  The two dot
// products run as four chains each.
__device__ __forceinline__ void dl_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void dl_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}

template <int L, int ROWS>
__global__ void __launch_bounds__(DL_THREADS) delta_scan_kernel(DeltaArgs p) {
    pdl_grid_sync();
    extern __shared__ __align__(16) float sm[];
    constexpr int COLS = DL_THREADS / L, DPAD = ROWS * L;
    const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.nh / p.nkv);
    const int d = p.d, dv = p.dv;
    const int l = threadIdx.x % L, jc = threadIdx.x / L;
    const int j = blockIdx.x * COLS + jc;           // the thread's column
    const bool live = j < dv;
    const int first = p.cu_q[b], n = p.cu_q[b + 1] - first;
    const int nq = p.nkv * d, C = 2 * nq + p.nh * dv;
    float* S_col = p.state + (size_t)p.slots[b] * p.state_elems + ((size_t)h * dv + (live ? j : 0)) * d;
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        const int i = 4 * (l + L * (r >> 2)) + (r & 3);
        S[r] = (live && i < d) ? S_col[i] : 0.f;
    }
    // Two buffers of a tile of tokens in shared memory: q, k, g [tile, DPAD] each, v [tile, COLS], beta [tile].  The next
    // tile is on its way (cp.async) while this one is computed.  The padding rows beyond d are written once.
    constexpr int BUF = DL_TILE * (3 * DPAD + COLS + 1);
    const int j0 = blockIdx.x * COLS;
    const float* __restrict__ qkv = p.qkv;
    const float* __restrict__ gg = p.g;
    float* __restrict__ out = p.out;
    if (d < DPAD)
        for (int e = threadIdx.x; e < 2 * DL_TILE * (DPAD - d); e += DL_THREADS) {
            const int bb = e / (DL_TILE * (DPAD - d)), r = e % (DL_TILE * (DPAD - d));
            const int at = (r / (DPAD - d)) * DPAD + d + r % (DPAD - d);
            sm[bb * BUF + at] = 0.f;
            sm[bb * BUF + DL_TILE * DPAD + at] = 0.f;
            sm[bb * BUF + 2 * DL_TILE * DPAD + at] = 1.f;
        }
    const bool wide = (d & 3) == 0 && (C & 3) == 0;          // rows of q, k and the decay start on 16-byte boundaries
    auto stage = [&](int buf, int t0) {
        float* sq = sm + buf * BUF;
        float* sk = sq + DL_TILE * DPAD;
        float* sg = sk + DL_TILE * DPAD;
        float* sv = sg + DL_TILE * DPAD;
        float* sb = sv + DL_TILE * COLS;
        const int nt = min(DL_TILE, n - t0);
        if (wide) {
            const int per_row = d >> 2;
            for (int e = threadIdx.x; e < nt * per_row; e += DL_THREADS) {
                const int tt = e / per_row, i = (e - tt * per_row) * 4;
                const size_t t = (size_t)(first + t0 + tt);
                dl_cp16(sq + tt * DPAD + i, qkv + t * C + (size_t)hk * d + i);
                dl_cp16(sk + tt * DPAD + i, qkv + t * C + nq + (size_t)hk * d + i);
                dl_cp16(sg + tt * DPAD + i, gg + t * p.nh * d + (size_t)h * d + i);
            }
        } else {
            for (int e = threadIdx.x; e < nt * d; e += DL_THREADS) {
                const int tt = e / d, i = e - tt * d;
                const size_t t = (size_t)(first + t0 + tt);
                dl_cp4(sq + tt * DPAD + i, qkv + t * C + (size_t)hk * d + i);
                dl_cp4(sk + tt * DPAD + i, qkv + t * C + nq + (size_t)hk * d + i);
                dl_cp4(sg + tt * DPAD + i, gg + t * p.nh * d + (size_t)h * d + i);
            }
        }
        for (int e = threadIdx.x; e < nt * COLS; e += DL_THREADS) {
            const int tt = e / COLS, c = e - tt * COLS;
            if (j0 + c < dv) dl_cp4(sv + e, qkv + (size_t)(first + t0 + tt) * C + 2 * nq + (size_t)h * dv + j0 + c);
        }
        for (int e = threadIdx.x; e < nt; e += DL_THREADS) dl_cp4(sb + e, p.beta + (size_t)(first + t0 + e) * p.nh + h);
    };
    if (n > 0) stage(0, 0);
    asm volatile("cp.async.commit_group;\n" ::);
    for (int t0 = 0, it = 0; t0 < n; t0 += DL_TILE, it++) {
        const int nt = min(DL_TILE, n - t0);
        if (t0 + DL_TILE < n) stage((it + 1) & 1, t0 + DL_TILE);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();
        const float* sq = sm + (it & 1) * BUF;
        const float* sk = sq + DL_TILE * DPAD;
        const float* sg = sk + DL_TILE * DPAD;
        const float* sv = sg + DL_TILE * DPAD;
        const float* sb = sv + DL_TILE * COLS;
        for (int tt = 0; tt < nt; tt++) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DPAD);
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * DPAD);
            const float4* g4 = reinterpret_cast<const float4*>(sg + tt * DPAD);
            float4 kk[ROWS / 4], qq[ROWS / 4];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS / 4; r++) {
                kk[r] = k4[l + L * r];
                qq[r] = q4[l + L * r];           // read now, used after the first reduction
            }
#pragma unroll
            for (int r = 0; r < ROWS / 4; r++) {
                const float4 g = g4[l + L * r];
                S[4 * r] *= g.x;
                S[4 * r + 1] *= g.y;
                S[4 * r + 2] *= g.z;
                S[4 * r + 3] *= g.w;
                a0 = fmaf(kk[r].x, S[4 * r], a0);
                a1 = fmaf(kk[r].y, S[4 * r + 1], a1);
                a2 = fmaf(kk[r].z, S[4 * r + 2], a2);
                a3 = fmaf(kk[r].w, S[4 * r + 3], a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float u = sb[tt] * (sv[tt * COLS + jc] - acc);
            a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS / 4; r++) {
                const float4 q = qq[r];
                S[4 * r] = fmaf(kk[r].x, u, S[4 * r]);
                S[4 * r + 1] = fmaf(kk[r].y, u, S[4 * r + 1]);
                S[4 * r + 2] = fmaf(kk[r].z, u, S[4 * r + 2]);
                S[4 * r + 3] = fmaf(kk[r].w, u, S[4 * r + 3]);
                a0 = fmaf(q.x, S[4 * r], a0);
                a1 = fmaf(q.y, S[4 * r + 1], a1);
                a2 = fmaf(q.z, S[4 * r + 2], a2);
                a3 = fmaf(q.w, S[4 * r + 3], a3);
            }
            float oacc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) oacc += __shfl_xor_sync(0xffffffffu, oacc, o);
            if (live && l == 0) out[(size_t)(first + t0 + tt) * p.nh * dv + (size_t)h * dv + j] = oacc;
        }
        __syncthreads();          // the tile after the next one goes into this buffer
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            const int i = 4 * (l + L * (r >> 2)) + (r & 3);
            if (i < d) S_col[i] = S[r];
        }
    }
}

extern "C" int illm_delta_rule_supported(int d, int dv, int taps) { return d >= 1 && d <= 16 * DL_ROWS && dv >= 1 && taps >= 1 && taps <= 64; }

template <int L, int ROWS>
static void launch_scan(const DeltaArgs& p, int B, int n_sms, cudaStream_t s) {
    constexpr int COLS = DL_THREADS / L;
    size_t smem = (size_t)(2 * DL_TILE * (3 * ROWS * L + COLS + 1)) * sizeof(float);
    // The scan is bound by what an SM's shared memory delivers per clock, so its blocks must spread over the SMs.  Launched
    // behind kernels that still hold most SMs, a small grid would be packed onto the few SMs that are free first (measured: 32
    // blocks, 2.5 ms instead of 0.95 ms).  Asking for more shared memory than the tiles need caps the blocks per SM at what an
    // even spread gives.
    const long long blocks = (long long)((p.dv + COLS - 1) / COLS) * p.nh * B;
    const long long per_sm = (blocks + n_sms - 1) / n_sms;
    if (per_sm < 5) {
        const size_t spread = (size_t)(220 * 1024) / (size_t)per_sm - 2048;
        smem = smem > spread ? smem : (spread < (size_t)200 * 1024 ? spread : (size_t)200 * 1024);
    }
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(delta_scan_kernel<L, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    illm_launch(delta_scan_kernel<L, ROWS>, dim3((p.dv + COLS - 1) / COLS, p.nh, B), dim3(DL_THREADS), smem, s, p);
}

// A column's rows over L lanes of 32 rows each, or, while the grid of ONE sequence then still fits the SMs once, over 2 L
// lanes of 16 rows or 4 L lanes of 8: a sequence's tokens are a chain, and fewer rows per thread shorten every link of it
// (one prompt of 2,048 tokens, 8 heads of 128 x 128: 0.78 / 0.62 ms with 32 / 16 rows; with two blocks on an SM the
// shorter rows gain nothing).  The choice does not depend on the batch, or a row's bits would.
template <int L>
static void launch_scan_for(const DeltaArgs& p, int B, cudaStream_t s) {
    static int n_sms = 0;
    if (!n_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        if (n_sms <= 0) n_sms = 1;
    }
    constexpr int L2 = 2 * L <= 32 ? 2 * L : L, L4 = 4 * L <= 32 ? 4 * L : L2;
    auto blocks_of = [&](int lanes) { return (long long)((p.dv + DL_THREADS / lanes - 1) / (DL_THREADS / lanes)) * p.nh; };
    if (L4 != L2 && blocks_of(L4) <= n_sms) launch_scan<L4, 8>(p, B, n_sms, s);
    else if (L2 != L && blocks_of(L2) <= n_sms) launch_scan<L2, 16>(p, B, n_sms, s);
    else launch_scan<L, 32>(p, B, n_sms, s);
}

// x: [T, ld] float32 with q at q_off (nkv * d columns), k at k_off, v at v_off (nh * dv), beta's logits at b_off (nh).
// state: float32 [slots, state_elems], state_elems >= nh * d * dv + (taps - 1) * (2 nkv d + nh dv).
// Scratch qkv [T, 2 nkv d + nh dv], g [T, nh d], beta [T, nh]; out [T, nh dv].
extern "C" int illm_delta_rule(const float* x, int T, int ld, int q_off, int k_off, int v_off, int b_off, const float* a, int nh, int nkv, int d,
                               int dv, int taps, const float* conv_q, const float* conv_k, const float* conv_v, const float* a_log,
                               const float* dt_bias, float q_scale, float* state, long long state_elems, const int* slots, const int* cu_q,
                               const int* token_pos, const int* token_seq, const int* seq_lens, float* qkv, float* g, float* beta, float* out,
                               int B, void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if (!illm_delta_rule_supported(d, dv, taps) || nkv <= 0 || nh % nkv) return ILLM_ERR_BAD_ARG;
    const long long C = 2LL * nkv * d + (long long)nh * dv;
    if (state_elems < (long long)nh * d * dv + (taps - 1) * C) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    DeltaArgs p;
    p.x = x; p.T = T; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.b_off = b_off;
    p.a = a; p.nh = nh; p.nkv = nkv; p.d = d; p.dv = dv; p.taps = taps;
    p.conv_q = conv_q; p.conv_k = conv_k; p.conv_v = conv_v; p.a_log = a_log; p.dt_bias = dt_bias; p.q_scale = q_scale;
    p.state = state; p.state_elems = state_elems; p.slots = slots; p.cu_q = cu_q; p.token_pos = token_pos; p.token_seq = token_seq;
    p.seq_lens = seq_lens; p.qkv = qkv; p.g = g; p.beta = beta; p.out = out;
    const int hpb = d > 256 ? 1 : 256 / ((d + 31) / 32 * 32);
    const long long units = (2LL * nkv + hpb - 1) / hpb + ((long long)nh * dv + 1023) / 1024 + ((long long)nh * d + 1023) / 1024 + 1;
    if (units > 65535) return ILLM_ERR_BAD_ARG;
    p.prep_tokens = T >= 512 ? DL_PREP_TOKENS : 1;
    const dim3 pgrid((T + p.prep_tokens - 1) / p.prep_tokens, (unsigned)units);
    if (taps == 1) illm_launch(delta_prep_kernel<1>, pgrid, dim3(256), 0, s, p);
    else if (taps == 2) illm_launch(delta_prep_kernel<2>, pgrid, dim3(256), 0, s, p);
    else if (taps == 3) illm_launch(delta_prep_kernel<3>, pgrid, dim3(256), 0, s, p);
    else if (taps == 4) illm_launch(delta_prep_kernel<4>, pgrid, dim3(256), 0, s, p);
    else illm_launch(delta_prep_kernel<0>, pgrid, dim3(256), 0, s, p);
    if (taps > 1) illm_launch(conv_state_kernel, dim3((unsigned)((C + 127) / 128), B), dim3(128), 0, s, p);
    if (d <= 32) launch_scan_for<1>(p, B, s);
    else if (d <= 64) launch_scan_for<2>(p, B, s);
    else if (d <= 128) launch_scan_for<4>(p, B, s);
    else if (d <= 256) launch_scan_for<8>(p, B, s);
    else launch_scan_for<16>(p, B, s);
    return illm_launch_status();
}
