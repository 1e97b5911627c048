// The gated delta rule with a decay per head and key channel over a per-sequence state: the mixer "channel_delta".
//
//     q, k = silu(conv(W_q h)), silu(conv(W_k h))  [kv_heads x d],   v = silu(conv(W_v h))  [heads x dv]
//     q, k made unit vectors per head, q times q_scale;   beta = sigmoid(W_b h)  [heads]
//     g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias))  [heads x d]
//     per head:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          (float32)
//     y = W_o ( rmsnorm_per_head(o) * w_norm * sigmoid(W_g2 (W_g1 h)) )
//
// conv is a causal convolution over time per channel (`conv` taps, the last the token's own).  Value head j reads
// query/key head j / (heads / kv_heads).  The state [heads, dv, d] float32 and the last conv - 1 rows of the raw
// q, k, v projections form the layer's cache entry (FixedState), zero when a sequence starts; a step of any
// number of tokens continues from it.  The two low ranks (of W_a1 and W_g1) are parameters (`a_rank`, `g_rank`) or,
// when not given, the shapes of those tensors in the weight file.  Everything between the projections and the
// normed, gated row is float32 in both modes.
#include <cmath>

#include "parts/parts.h"

namespace illm {

namespace {

struct ChannelDelta : Mixer {
    long long hidden;
    int n_heads, n_kv_heads, head_dim, v_head_dim, taps;
    long long a_rank, g_rank;
    float norm_eps, q_scale;
    bool out_f32;
    std::map<std::string, std::string> names;
    DeviceBuffer w_buf;
    Mat w_in;
    OwnedMat w_a_up, w_g_up, w_o, conv_q, conv_k, conv_v, a_log, dt_bias, norm_w;

    ChannelDelta(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")),
              n_kv_heads((int)s.get_int("n_kv_heads", s.get_int("n_heads"))), head_dim((int)s.get_int("head_dim")),
              v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))), taps((int)s.get_int("conv", 1)), a_rank(s.get_int("a_rank", 0)),
              g_rank(s.get_int("g_rank", 0)), norm_eps((float)s.get_double("norm_eps", 1e-6)),
              q_scale((float)s.get_double("q_scale", 1.0 / std::sqrt((double)s.get_int("head_dim")))),
              out_f32(s.get_string("output_dtype", "compute") == "float32") {
        if (hidden <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || v_head_dim <= 0 || taps < 1 || a_rank < 0 || g_rank < 0)
            throw ConfigError("channel_delta: sizes must be positive");
        if (n_heads % n_kv_heads) throw ConfigError("channel_delta: n_heads must be a multiple of n_kv_heads");
        names = {{"q", "q_proj.weight"}, {"k", "k_proj.weight"}, {"v", "v_proj.weight"}, {"q_conv", "q_conv.weight"}, {"k_conv", "k_conv.weight"},
                 {"v_conv", "v_conv.weight"}, {"beta", "b_proj.weight"}, {"a_log", "A_log"}, {"norm", "norm.weight"}, {"a_down", "a_down.weight"},
                 {"a_up", "a_up.weight"}, {"dt_bias", "dt_bias"}, {"g_down", "g_down.weight"}, {"g_up", "g_up.weight"}, {"o", "o_proj.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
        if (rt && !ops::delta_rule_supported(head_dim, v_head_dim, taps))
            throw ConfigError("channel_delta: a head of " + std::to_string(head_dim) + " key channels with " + std::to_string(taps) +
                              " taps is beyond the kernel (up to 512 channels, 64 taps)");
    }
    bool graph_safe() const override { return true; }      // everything that varies is read on the device
    bool pad_safe() const override { return false; }       // tokens behind the real ones would enter the state
    CacheRequest cache_request() const override {
        return CacheRequest::state({ops::delta_rule_state_elements(n_heads, n_kv_heads, head_dim, v_head_dim, taps)}, DType::F32);
    }
    long long qk_rows() const { return (long long)n_kv_heads * head_dim; }
    long long v_rows() const { return (long long)n_heads * v_head_dim; }
    long long g_rows() const { return (long long)n_heads * head_dim; }
    TensorDecls tensors() const override {
        // a rank that is not given is whatever the file has (-1 matches any size)
        const long long ra = a_rank > 0 ? a_rank : -1, rg = g_rank > 0 ? g_rank : -1;
        auto nm = [&](const char* role) { return names.at(role); };
        return {{nm("q"), TensorDecl{{qk_rows(), hidden}}}, {nm("q_conv"), TensorDecl{{qk_rows(), (long long)taps}}},
                {nm("k"), TensorDecl{{qk_rows(), hidden}}}, {nm("k_conv"), TensorDecl{{qk_rows(), (long long)taps}}},
                {nm("v"), TensorDecl{{v_rows(), hidden}}}, {nm("v_conv"), TensorDecl{{v_rows(), (long long)taps}}},
                {nm("beta"), TensorDecl{{(long long)n_heads, hidden}}}, {nm("a_log"), TensorDecl{{(long long)n_heads}}},
                {nm("norm"), TensorDecl{{(long long)v_head_dim}, "norm"}}, {nm("a_down"), TensorDecl{{ra, hidden}}},
                {nm("a_up"), TensorDecl{{g_rows(), ra}}}, {nm("dt_bias"), TensorDecl{{g_rows()}}}, {nm("g_down"), TensorDecl{{rg, hidden}}},
                {nm("g_up"), TensorDecl{{v_rows(), rg}}}, {nm("o"), TensorDecl{{hidden, v_rows()}}}};
    }
    long long off_v() const { return 2 * qk_rows(); }
    long long off_b() const { return off_v() + v_rows(); }
    long long off_a() const { return off_b() + n_heads; }
    long long off_g() const { return off_a() + a_rank; }
    void load(TensorSource& src) override {
        a_rank = src.shape(names.at("a_down")).at(0);
        g_rank = src.shape(names.at("g_down")).at(0);
        if (a_rank <= 0 || g_rank <= 0) throw ConfigError("channel_delta: a model made from random numbers needs a_rank and g_rank");
        if (src.shape(names.at("a_up")).at(1) != a_rank || src.shape(names.at("g_up")).at(1) != g_rank)
            throw WeightError("channel_delta: the two halves of a low-rank projection differ in rank");
        const long long all = off_g() + g_rank;
        const size_t es = dtype_size(rt->dtype);
        w_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed projections of a delta-rule layer");
        w_in = Mat{w_buf.get(), all, hidden, rt->dtype, all};
        char* p = (char*)w_in.p;
        auto at = [&](long long row) { return p + (size_t)row * hidden * es; };
        src.fetch_into(names.at("q"), at(0), rt->dtype);
        src.fetch_into(names.at("k"), at(qk_rows()), rt->dtype);
        src.fetch_into(names.at("v"), at(off_v()), rt->dtype);
        src.fetch_into(names.at("beta"), at(off_b()), rt->dtype);
        src.fetch_into(names.at("a_down"), at(off_a()), rt->dtype);
        src.fetch_into(names.at("g_down"), at(off_g()), rt->dtype);
        w_a_up = fetch_owned(rt, src, names.at("a_up"), rt->dtype, "a delta-rule layer's decay matrix");
        w_g_up = fetch_owned(rt, src, names.at("g_up"), rt->dtype, "a delta-rule layer's gate matrix");
        w_o = fetch_owned(rt, src, names.at("o"), rt->dtype, "the output matrix of a delta-rule layer");
        // what the recurrence's preparation reads is float32
        conv_q = fetch_owned(rt, src, names.at("q_conv"), DType::F32, "a convolution's taps");
        conv_k = fetch_owned(rt, src, names.at("k_conv"), DType::F32, "a convolution's taps");
        conv_v = fetch_owned(rt, src, names.at("v_conv"), DType::F32, "a convolution's taps");
        a_log = fetch_owned(rt, src, names.at("a_log"), DType::F32, "a delta-rule layer's decay rates");
        dt_bias = fetch_owned(rt, src, names.at("dt_bias"), DType::F32, "a delta-rule layer's decay bias");
        norm_w = fetch_owned(rt, src, names.at("norm"), DType::F32, "a delta-rule layer's norm weight");
    }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::State) throw EngineError("channel_delta: the layer's cache entry holds no state");
        if (!writes) throw EngineError("channel_delta: the state belongs to one layer");
        Device& dev = *rt->dev;
        Mat x = ops::linear(dev, rt->gemm, h, w_in, DType::F32, false).m;
        Mat a = ops::linear(dev, rt->gemm, ops::take_columns(dev, x, off_a(), a_rank, rt->dtype), w_a_up.m, DType::F32, false).m;
        Mat gz = ops::linear(dev, rt->gemm, ops::take_columns(dev, x, off_g(), g_rank, rt->dtype), w_g_up.m, DType::F32, false).m;
        ops::DeltaRule p;
        p.q_off = 0;
        p.k_off = (int)qk_rows();
        p.v_off = (int)off_v();
        p.b_off = (int)off_b();
        p.n_heads = n_heads;
        p.n_kv_heads = n_kv_heads;
        p.head_dim = head_dim;
        p.v_head_dim = v_head_dim;
        p.taps = taps;
        p.conv_q = (const float*)conv_q.m.p;
        p.conv_k = (const float*)conv_k.m.p;
        p.conv_v = (const float*)conv_v.m.p;
        p.a_log = (const float*)a_log.m.p;
        p.dt_bias = (const float*)dt_bias.m.p;
        p.q_scale = q_scale;
        Mat o = ops::delta_rule(dev, x, a, p, ctx, cache.st);
        Mat y = ops::group_norm_gate(dev, o, v_head_dim, (const float*)norm_w.m.p, norm_eps, (const float*)gz.p, (int)gz.cols, 2, rt->dtype,
                                     v_head_dim);
        return ops::linear(dev, rt->gemm, y, w_o.m, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

}  // namespace

void register_delta_parts(std::map<std::string, PartFactory<Mixer>>& mixers) {
    mixers["channel_delta"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new ChannelDelta(s, rt)); };
}

}  // namespace illm
