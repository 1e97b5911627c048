// Softmax attention through low-rank latents: the mixer "latent_attention".
//
//     c_q = rmsnorm(W_dq h) * w_q;   q_h = U_q,h c_q  [heads x d]
//     c   = rmsnorm(W_dkv h) * w_kv  [kv_rank]                    the only thing cached
//     k_h = U_k,h c,  v_h = U_v,h c;   score = (q_h . k_h) * scale over the visible positions (all before, or the
//     last `window`);   softmax;   y = W_o [sum_j p_j v_h,j]_h
//
// No position encoding.  It is computed in the absorbed form: score = (U_k,h^T q_h) . c and
// o_h = U_v,h (sum_j p_j c_j), so the attention kernels see ONE key/value head of kv_rank channels (the cached c is
// key and value at once: a keys-only cache entry) and `heads` query heads, and the per-head maps U_k,h^T and U_v,h run
// before and after them (ops::head_linear).  A step's keys and values are never expanded per head.
#include <cmath>

#include "parts/parts.h"

namespace illm {

namespace {

struct LatentAttention : Mixer {
    long long hidden;
    int n_heads, head_dim, v_head_dim, q_rank, kv_rank, window;
    float scale, norm_eps;
    bool out_f32;
    std::map<std::string, std::string> names;
    DeviceBuffer w_buf;
    Mat w_down;
    OwnedMat w_uq, w_uk, w_uv, w_o, n_q, n_kv;

    LatentAttention(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), head_dim((int)s.get_int("head_dim")),
              v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))), q_rank((int)s.get_int("q_rank")), kv_rank((int)s.get_int("kv_rank")),
              window((int)s.get_int("window", 0)), norm_eps((float)s.get_double("norm_eps", 1e-6)),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (hidden <= 0 || n_heads <= 0 || head_dim <= 0 || v_head_dim <= 0 || q_rank <= 0 || kv_rank <= 0 || window < 0)
            throw ConfigError("latent_attention: sizes must be positive");
        scale = s.has("scale") ? (float)s.get_double("scale") : (float)(1.0 / std::sqrt((double)head_dim));
        names = {{"q_down", "q_a_proj.weight"}, {"q_norm", "q_a_norm.weight"}, {"q_up", "q_b_proj.weight"}, {"kv_down", "kv_a_proj.weight"},
                 {"kv_norm", "kv_a_norm.weight"}, {"k_up", "k_b_proj.weight"}, {"v_up", "v_b_proj.weight"}, {"o", "o_proj.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
        if (rt && kv_rank > 1024) throw ConfigError("latent_attention: a latent of " + std::to_string(kv_rank) + " channels is beyond the kernels (up to 1024)");
    }
    bool graph_safe() const override { return true; }
    bool pad_safe() const override { return false; }
    CacheRequest cache_request() const override { return CacheRequest::paged_keys_only(1, kv_rank, window); }
    TensorDecls tensors() const override {
        const long long q = (long long)n_heads * head_dim, v = (long long)n_heads * v_head_dim;
        auto nm = [&](const char* role) { return names.at(role); };
        return {{nm("q_down"), TensorDecl{{(long long)q_rank, hidden}}}, {nm("q_norm"), TensorDecl{{(long long)q_rank}, "norm"}},
                {nm("q_up"), TensorDecl{{q, (long long)q_rank}}}, {nm("kv_down"), TensorDecl{{(long long)kv_rank, hidden}}},
                {nm("kv_norm"), TensorDecl{{(long long)kv_rank}, "norm"}}, {nm("k_up"), TensorDecl{{q, (long long)kv_rank}}},
                {nm("v_up"), TensorDecl{{v, (long long)kv_rank}}}, {nm("o"), TensorDecl{{hidden, v}}}};
    }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        const long long all = (long long)q_rank + kv_rank;
        w_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed latent projections");
        w_down = Mat{w_buf.get(), all, hidden, rt->dtype, all};
        src.fetch_into(names.at("q_down"), w_down.p, rt->dtype);
        src.fetch_into(names.at("kv_down"), (char*)w_down.p + (size_t)q_rank * hidden * es, rt->dtype);
        w_uq = fetch_owned(rt, src, names.at("q_up"), rt->dtype, "the query up-projection");
        w_uk = fetch_owned(rt, src, names.at("k_up"), rt->dtype, "the key up-projection");
        w_uv = fetch_owned(rt, src, names.at("v_up"), rt->dtype, "the value up-projection");
        w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of an attention layer");
        n_q = fetch_owned(rt, src, names.at("q_norm"), DType::F32, "a latent norm's weight");
        n_kv = fetch_owned(rt, src, names.at("kv_norm"), DType::F32, "a latent norm's weight");
    }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::KV) throw EngineError("latent_attention: the layer's cache entry holds no keys");
        Device& dev = *rt->dev;
        KVView kv = cache.kv;
        kv.writes = writes;
        if (kv.n_kv_heads != 1 || kv.head_dim != kv_rank) throw EngineError("latent_attention: the cache entry does not hold this layer's latent");
        Mat x = ops::linear(dev, rt->gemm, h, w_down, DType::F32, false).m;
        Mat cq = ops::latent_prep(dev, x, q_rank, kv_rank, (const float*)n_q.m.p, (const float*)n_kv.m.p, norm_eps, ctx, kv, rt->dtype);
        // a prompt's queries are rounded to the activation dtype for the library's batched product; single tokens stay float32
        Mat q = ops::linear(dev, rt->gemm, cq, w_uq.m, ctx.is_decode ? DType::F32 : rt->dtype, false).m;
        Mat qa = ops::head_linear(dev, q, w_uk.m, n_heads, true, rt->dtype);          // U_k,h^T q_h
        const ops::Geometry g{n_heads, 1, kv_rank};
        ops::AttentionExtras ex;
        ex.wide_weights = true;       // the softmax weights are not to be rounded to eight bits
        // a latent whose width the framework's attention kernels do not take (not a multiple of 8, beyond 256) has a plain kernel
        Mat o = (kv_rank % 8 || kv_rank > ops::kMaxHeadDimGeneric) ? ops::latent_attention_any(dev, qa, kv, ctx, n_heads, scale)
                                                                  : ops::attention_ex(dev, qa, kv, ctx, g, scale, ex);
        Mat ov = ops::head_linear(dev, o, w_uv.m, n_heads, false, rt->dtype);         // U_v,h (sum p c)
        return ops::linear(dev, rt->gemm, ov, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

}  // namespace

void register_latent_parts(std::map<std::string, PartFactory<Mixer>>& mixers) {
    mixers["latent_attention"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new LatentAttention(s, rt)); };
}

}  // namespace illm
