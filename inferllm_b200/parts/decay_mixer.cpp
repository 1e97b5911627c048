// Linear attention with a fixed decay per head over a per-sequence state: the mixer
// "decay_linear_attention".
//
//     q, k = act(W_q h), act(W_k h)  [heads x d],   v = act_v(W_v h)  [heads x dv]
//     q, k rotated by the position (optional, a rotate-half table rotation);  k = k * k_scale
//     S_t = decay_h S_{t-1} + k_t v_t^T;   o_t = S_t^T q_t                      (per head, float32)
//     y = W_o ( norm(o) * gate_act(W_g h) )
//
// with norm either one RMS norm with a weight over all heads together ("joint") or an RMS norm
// without a weight per head ("per_head").  Everything from the float32 projection to the normed,
// gated row is float32.  The state [heads, d, dv] float32 is the layer's cache entry (FixedState),
// zero when a sequence starts; a step of any number of tokens continues from it.  Two known layer
// kinds are settings of this one part: silu on q, k, v, no rotation, joint norm and a sigmoid gate;
// or no activation, rotated q and k with k scaled by d^(-1/2), per-head norm and a silu gate.
#include <cmath>

#include "parts/parts.h"

namespace illm {

namespace {

struct DecayLinearAttention : Mixer {
    long long hidden;
    int n_heads, head_dim, v_head_dim;
    int qk_act, v_act, gate_act;
    bool joint_norm, out_f32;
    float k_scale, norm_eps;
    std::vector<float> decay;
    std::map<std::string, std::string> names;
    std::unique_ptr<PositionEncoding> position;
    DeviceBuffer w_buf, o_buf, decay_buf;
    Mat w_all, w_o;
    OwnedMat norm_w;

    static int act_code(const PartSpec& s, const char* key, const char* fallback) {
        const std::string a = s.get_string(key, fallback);
        if (a == "none") return 0;
        if (a == "silu") return 1;
        if (a == "sigmoid") return 2;
        throw ConfigError("decay_linear_attention: " + std::string(key) + " '" + a + "' is not supported (none, silu, sigmoid)");
    }

    DecayLinearAttention(const PartSpec& s, Runtime* rt)
            : Mixer(s, rt), hidden(s.get_int("hidden_size")), n_heads((int)s.get_int("n_heads")), head_dim((int)s.get_int("head_dim")),
              v_head_dim((int)s.get_int("v_head_dim", s.get_int("head_dim"))), qk_act(act_code(s, "qk_activation", "none")),
              v_act(act_code(s, "v_activation", "none")), gate_act(act_code(s, "gate_activation", "sigmoid")),
              joint_norm(s.get_string("out_norm", "joint") == "joint"), out_f32(s.get_string("output_dtype", "compute") == "float32"),
              k_scale((float)s.get_double("k_scale", 1.0)), norm_eps((float)s.get_double("norm_eps", 1e-6)) {
        if (hidden <= 0 || n_heads <= 0 || head_dim <= 0 || v_head_dim <= 0) throw ConfigError("decay_linear_attention: sizes must be positive");
        const std::string on = s.get_string("out_norm", "joint");
        if (on != "joint" && on != "per_head") throw ConfigError("decay_linear_attention: out_norm '" + on + "' is not supported (joint, per_head)");
        if (qk_act == 2 || v_act == 2 || gate_act == 0)
            throw ConfigError("decay_linear_attention: q, k, v take none or silu; the gate takes silu or sigmoid");
        if (!s.has("decay") || !s.params.at("decay").is_array() || (int)s.params.at("decay").size() != n_heads)
            throw ConfigError("decay_linear_attention: 'decay' must list one number per head");
        for (const Json& d : s.params.at("decay").items()) {
            if (!d.is_number()) throw ConfigError("decay_linear_attention: 'decay' must list numbers");
            decay.push_back((float)d.as_double());
        }
        names = {{"q", "q_proj.weight"}, {"k", "k_proj.weight"}, {"v", "v_proj.weight"}, {"gate", "g_proj.weight"}, {"o", "o_proj.weight"},
                 {"norm", "norm.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
        if (rt && !ops::decay_scan_supported(head_dim, v_head_dim))
            throw ConfigError("decay_linear_attention: a state of " + std::to_string(head_dim) + " x " + std::to_string(v_head_dim) +
                              " per head is beyond the kernel (head sizes up to 1024)");
        position = build_position(s.has("position") ? s.get_part("position") : PartSpec("none", Json::object()), rt);
        if (rt) position->prepare();
    }
    bool graph_safe() const override { return true; }      // everything that varies is read on the device
    bool pad_safe() const override { return false; }       // tokens behind the real ones would enter the state
    CacheRequest cache_request() const override { return CacheRequest::state({n_heads, head_dim, v_head_dim}, DType::F32); }

    long long qk_rows() const { return (long long)n_heads * head_dim; }
    long long v_rows() const { return (long long)n_heads * v_head_dim; }
    TensorDecls tensors() const override {
        TensorDecls d = {{names.at("q"), TensorDecl{{qk_rows(), hidden}}}, {names.at("k"), TensorDecl{{qk_rows(), hidden}}},
                         {names.at("v"), TensorDecl{{v_rows(), hidden}}}, {names.at("gate"), TensorDecl{{v_rows(), hidden}}},
                         {names.at("o"), TensorDecl{{hidden, v_rows()}}}};
        if (joint_norm) d.push_back({names.at("norm"), TensorDecl{{v_rows()}, "norm"}});
        return d;
    }
    void load(TensorSource& src) override {
        const long long all = 2 * qk_rows() + 2 * v_rows();
        const size_t es = dtype_size(rt->dtype);
        w_buf = DeviceBuffer(rt->dev, (size_t)all * hidden * es, "the packed projections of a linear-attention layer");
        w_all = Mat{w_buf.get(), all, hidden, rt->dtype, all};
        char* p = (char*)w_all.p;
        src.fetch_into(names.at("q"), p, rt->dtype);
        src.fetch_into(names.at("k"), p + (size_t)qk_rows() * hidden * es, rt->dtype);
        src.fetch_into(names.at("v"), p + (size_t)2 * qk_rows() * hidden * es, rt->dtype);
        src.fetch_into(names.at("gate"), p + (size_t)(2 * qk_rows() + v_rows()) * hidden * es, rt->dtype);
        o_buf = DeviceBuffer(rt->dev, (size_t)hidden * v_rows() * es, "the output matrix of a linear-attention layer");
        w_o = Mat{o_buf.get(), hidden, v_rows(), rt->dtype, hidden};
        src.fetch_into(names.at("o"), w_o.p, rt->dtype);
        if (joint_norm) norm_w = fetch_owned(rt, src, names.at("norm"), DType::F32, "a linear-attention layer's norm weight");
        decay_buf = DeviceBuffer(rt->dev, decay.size() * sizeof(float), "the decays of a linear-attention layer");
        rt->dev->synchronize();
        check_cuda(cudaMemcpy(decay_buf.get(), decay.data(), decay.size() * sizeof(float), cudaMemcpyHostToDevice), "uploading the decays");
    }

    MatOrPartials forward(const Mat& h, const StepContext& ctx, const CacheView& cache, bool writes, bool may_defer) override {
        if (cache.kind != CacheView::State) throw EngineError("decay_linear_attention: the layer's cache entry holds no state");
        if (!writes) throw EngineError("decay_linear_attention: the state belongs to one layer");
        Device& dev = *rt->dev;
        Mat x = ops::linear(dev, rt->gemm, h, w_all, DType::F32, false).m;
        ops::DecayScan p;
        p.q_off = 0;
        p.k_off = (int)qk_rows();
        p.v_off = (int)(2 * qk_rows());
        p.n_heads = n_heads;
        p.head_dim = head_dim;
        p.v_head_dim = v_head_dim;
        p.qk_act = qk_act;
        p.v_act = v_act;
        p.k_scale = k_scale;
        p.decay = (const float*)decay_buf.get();
        p.in_order = rt->is_f32();      // the float32 mode gives the same bits however a prompt is cut
        const float* table = nullptr;
        int rot = 0;
        long long n_pos = 0;
        if (!position->rotation_table(&table, &rot, &n_pos))
            throw EngineError("decay_linear_attention: the position encoding must be none or a rotate-half table rotation");
        p.cos_sin = table;
        p.rot_dim = rot;
        p.n_pos = n_pos;
        Mat o = ops::decay_scan(dev, x, p, ctx, cache.st);
        const float* gate = (const float*)x.p + (2 * qk_rows() + v_rows());
        Mat y = ops::group_norm_gate(dev, o, joint_norm ? (int)v_rows() : v_head_dim, joint_norm ? (const float*)norm_w.m.p : nullptr, norm_eps,
                                     gate, (int)x.cols, gate_act, rt->dtype);
        return ops::linear(dev, rt->gemm, y, w_o, out_f32 ? DType::F32 : rt->dtype, may_defer);
    }
};

}  // namespace

void register_decay_parts(std::map<std::string, PartFactory<Mixer>>& mixers) {
    mixers["decay_linear_attention"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<Mixer>(new DecayLinearAttention(s, rt)); };
}

}  // namespace illm
