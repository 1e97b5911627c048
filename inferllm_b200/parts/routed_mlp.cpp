// Routed feed-forward (mixture of experts): the feed-forward "routed_mlp".
//
//     z = W_r h (+ b_r)  [experts], float32;   the `top` experts with the largest z;   weights = softmax over the chosen z
//     y = sum over the chosen experts of weight * W_down,e ( act(W_gate,e h) * (W_up,e h) )
//
// Experts have no biases.  Their matrices are packed at load: gate and up rows of an expert in turn (row 2i the gate
// row and row 2i + 1 the up row of output i, so that a product's epilogue can apply the activation) in one
// [experts * 2 ff, hidden] matrix, the down matrices in one [experts * hidden, ff].  The tokens of a step are
// grouped by expert on the device (nothing of the routing comes back to the host), so a step launches the same
// kernels whatever the router decides.  Tensor names: `names` gives "router", "router_bias", the experts' prefix
// "expert" (followed by the expert's number and a dot) and "gate", "up", "down" below it.
#include "parts/parts.h"

namespace illm {

namespace {

struct RoutedMLP : FeedForward {
    long long hidden, inter;
    int experts, top, act;
    bool has_bias;
    std::map<std::string, std::string> names;
    DeviceBuffer gu_buf, down_buf;
    Mat w_gate_up, w_down;
    OwnedMat w_router, b_router;

    RoutedMLP(const PartSpec& s, Runtime* rt)
            : FeedForward(s, rt), hidden(s.get_int("hidden_size")), inter(s.get_int("intermediate_size")), experts((int)s.get_int("experts")),
              top((int)s.get_int("top")), act(ops::gate_act_from_name(s.get_string("activation", "silu"))), has_bias(s.get_bool("router_bias", false)) {
        if (hidden <= 0 || inter <= 0 || experts <= 0 || top <= 0 || top > experts)
            throw ConfigError("routed_mlp: sizes must be positive and top at most the number of experts");
        if (act < 0) throw ConfigError("routed_mlp: activation '" + s.get_string("activation", "silu") + "' is not supported (silu, relu, gelu_tanh)");
        names = {{"router", "router.weight"}, {"router_bias", "router.bias"}, {"expert", "experts."}, {"gate", "gate_proj.weight"},
                 {"up", "up_proj.weight"}, {"down", "down_proj.weight"}};
        if (s.has("names"))
            for (auto& m : s.params.at("names").members()) names[m.first] = m.second.as_string();
    }
    std::string expert_tensor(int e, const char* role) const { return names.at("expert") + std::to_string(e) + "." + names.at(role); }
    TensorDecls tensors() const override {
        TensorDecls d = {{names.at("router"), TensorDecl{{(long long)experts, hidden}}}};
        if (has_bias) d.push_back({names.at("router_bias"), TensorDecl{{(long long)experts}}});
        for (int e = 0; e < experts; e++) {
            d.push_back({expert_tensor(e, "gate"), TensorDecl{{inter, hidden}}});
            d.push_back({expert_tensor(e, "up"), TensorDecl{{inter, hidden}}});
            d.push_back({expert_tensor(e, "down"), TensorDecl{{hidden, inter}}});
        }
        return d;
    }
    void load(TensorSource& src) override {
        const size_t es = dtype_size(rt->dtype);
        w_router = fetch_owned(rt, src, names.at("router"), rt->dtype, "a router's matrix");
        if (has_bias) b_router = fetch_owned(rt, src, names.at("router_bias"), DType::F32, "a router's bias");
        gu_buf = DeviceBuffer(rt->dev, (size_t)experts * 2 * inter * hidden * es, "the experts' packed gate/up matrices");
        down_buf = DeviceBuffer(rt->dev, (size_t)experts * hidden * inter * es, "the experts' down matrices");
        w_gate_up = Mat{gu_buf.get(), (long long)experts * 2 * inter, hidden, rt->dtype, (long long)experts * 2 * inter};
        w_down = Mat{down_buf.get(), (long long)experts * hidden, inter, rt->dtype, (long long)experts * hidden};
        for (int e = 0; e < experts; e++) {
            char* gu = (char*)w_gate_up.p + (size_t)e * 2 * inter * hidden * es;
            src.fetch_into(expert_tensor(e, "gate"), gu, rt->dtype, 2 * hidden);              // rows 2i
            src.fetch_into(expert_tensor(e, "up"), gu + (size_t)hidden * es, rt->dtype, 2 * hidden);  // rows 2i + 1
            src.fetch_into(expert_tensor(e, "down"), (char*)w_down.p + (size_t)e * hidden * inter * es, rt->dtype);
        }
    }
    MatOrPartials forward(const Mat& h, const StepContext&, bool) override {
        Device& dev = *rt->dev;
        Mat logits = ops::linear(dev, rt->gemm, h, w_router.m, DType::F32, false).m;
        MatOrPartials r;
        r.m = ops::moe_forward(dev, h, logits, has_bias ? (const float*)b_router.m.p : nullptr, experts, top, w_gate_up, w_down, act);
        return r;
    }
};

}  // namespace

void register_routed_parts(std::map<std::string, PartFactory<FeedForward>>& ffs) {
    ffs["routed_mlp"] = [](const PartSpec& s, Runtime* rt) { return std::unique_ptr<FeedForward>(new RoutedMLP(s, rt)); };
}

}  // namespace illm
