#include "config/vizosun.h"

#include <cmath>

namespace illm {

namespace {
const Json& need_obj(const Json& d, const std::string& key, const std::string& where) {
    if (!d.is_object() || !d.has(key) || !d.at(key).is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return d.at(key);
}
bool given(const Json& d, const std::string& key) { return d.is_object() && d.has(key) && !d.at(key).is_null(); }
Json obj(std::initializer_list<std::pair<const char*, Json>> kv) {
    Json o = Json::object();
    for (auto& p : kv) o.set(p.first, p.second);
    return o;
}
Json name_map(std::initializer_list<std::pair<const char*, const char*>> kv) {
    Json o = Json::object();
    for (auto& p : kv) o.set(p.first, std::string(p.second));
    return o;
}
}  // namespace

std::unique_ptr<ArchConfig> VizosunConfig::from_json(const Json& d) {
    std::unique_ptr<VizosunConfig> c(new VizosunConfig);
    c->raw = d;
    c->width = take_int(d, "width");
    c->vocab = take_int(d, "vocab");
    c->max_positions = take_int(d, "max_positions", 131072);
    c->norm_eps = take_double(need_obj(d, "norm", ""), "eps", 1e-6);
    if (c->width <= 0 || c->vocab <= 0 || c->max_positions <= 0) throw ConfigError("config.json: width, vocab and max_positions must be positive");
    if (!(c->norm_eps > 0)) throw ConfigError("config.json: norm.eps must be positive");
    if (!d.has("layers") || !d.at("layers").is_array() || d.at("layers").size() == 0)
        throw ConfigError("config.json: 'layers' must be a list with at least one layer");
    if (given(d, "embedding") && given(d.at("embedding"), "bigram")) {
        const Json& b = need_obj(d.at("embedding"), "bigram", "embedding: ");
        c->has_bigram = true;
        c->buckets = take_int(b, "buckets");
        c->mul_prev = take_int(b, "mul_prev");
        c->mul_cur = take_int(b, "mul_cur");
        if (c->buckets <= 0 || c->mul_prev < 0 || c->mul_cur < 0)
            throw ConfigError("config.json: embedding.bigram needs buckets > 0 and multipliers that are not negative");
    }
    if (given(d, "loop")) {
        const Json& l = need_obj(d, "loop", "");
        c->has_loop = true;
        c->loop_start = take_int(l, "start");
        c->loop_stop = take_int(l, "stop");
        c->loop_times = take_int(l, "times", 1);
        const long long n = (long long)d.at("layers").size();
        if (c->loop_start < 0 || c->loop_stop <= c->loop_start || c->loop_stop > n || c->loop_times < 1)
            throw ConfigError("config.json: loop needs 0 <= start < stop <= the number of layers and times >= 1");
    }
    c->model_spec();        // every layer is checked now, not at the first use
    return std::unique_ptr<ArchConfig>(c.release());
}

ModelSpec VizosunConfig::model_spec() const {
    ModelSpec s;
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = max_positions;
    const Json& layers = raw.at("layers");
    size_t i = 0;
    for (const Json& L : layers.items()) {
        const std::string where = "layer " + std::to_string(i) + ": ";
        if (!L.is_object()) throw ConfigError("config.json: " + where + "must be an object");
        const std::string type = take_string(L, "type", "");
        const Json& m = need_obj(L, "mixer", where);
        LayerSpec l;
        l.prefix = "l" + std::to_string(i) + ".";
        l.block = "parallel";
        l.names = {{"mixer", "mix."}, {"ffn", "mlp."}, {"norm1", "norm1"}};
        l.norms["norm1"] = PartSpec("rmsnorm", obj({{"size", width}, {"eps", norm_eps}, {"float32_weight", true}, {"tensor", std::string("")}}));
        const long long heads = take_int(m, "heads"), dim = take_int(m, "dim"), vdim = take_int(m, "vdim");
        if (heads <= 0 || dim <= 0 || vdim <= 0) throw ConfigError("config.json: " + where + "heads, dim and vdim must be positive");
        if (type == "channel_delta") {
            // the gated delta rule over a float32 state per head, with a decay per head and key channel from a low-rank
            // projection, short causal convolutions and silu on q, k, v, unit q and k, a sigmoid write strength per head,
            // and a per-head norm with a shared weight and a low-rank sigmoid gate on the way out
            const long long kvh = take_int(m, "kv_heads", heads), taps = take_int(m, "conv", 1);
            if (kvh <= 0 || heads % kvh) throw ConfigError("config.json: " + where + "heads must be a multiple of kv_heads");
            if (taps < 1) throw ConfigError("config.json: " + where + "conv must be at least 1");
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"n_kv_heads", kvh}, {"head_dim", dim}, {"v_head_dim", vdim},
                          {"conv", taps}, {"norm_eps", norm_eps}, {"q_scale", 1.0 / std::sqrt((double)dim)}, {"output_dtype", std::string("float32")},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"q_conv", "q.conv"}, {"k_conv", "k.conv"}, {"v_conv", "v.conv"},
                                              {"beta", "b"}, {"a_log", "A_log"}, {"norm", "norm"}, {"a_down", "a1"}, {"a_up", "a2"},
                                              {"dt_bias", "dt_bias"}, {"g_down", "g1"}, {"g_up", "g2"}, {"o", "o"}})}});
            // the two low ranks are the file's (the shapes of a1 and g1); a model made from random numbers names them
            if (given(m, "a_rank")) p.set("a_rank", take_int(m, "a_rank"));
            if (given(m, "g_rank")) p.set("g_rank", take_int(m, "g_rank"));
            l.mixer = PartSpec("channel_delta", p);
        } else if (type == "latent_attention") {
            // softmax attention without position encoding whose queries come out of a normed low-rank latent and whose keys
            // and values are maps of a second normed latent, the only thing cached; optionally over a sliding window
            const long long q_rank = take_int(m, "q_rank"), kv_rank = take_int(m, "kv_rank");
            if (q_rank <= 0 || kv_rank <= 0) throw ConfigError("config.json: " + where + "q_rank and kv_rank must be positive");
            long long window = 0;
            if (given(m, "mask")) {
                window = take_int(need_obj(m, "mask", where), "size", 0);
                if (window < 0) throw ConfigError("config.json: " + where + "mask.size must not be negative");
            }
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"head_dim", dim}, {"v_head_dim", vdim}, {"q_rank", q_rank},
                          {"kv_rank", kv_rank}, {"window", window}, {"scale", take_double(m, "scale", 1.0 / std::sqrt((double)dim))},
                          {"norm_eps", norm_eps}, {"output_dtype", std::string("float32")},
                          {"names", name_map({{"q_down", "dq"}, {"q_norm", "dq.norm"}, {"q_up", "uq"}, {"kv_down", "dkv"}, {"kv_norm", "dkv.norm"},
                                              {"k_up", "uk"}, {"v_up", "uv"}, {"o", "o"}})}});
            l.mixer = PartSpec("latent_attention", p);
        } else {
            throw ConfigError("config.json: " + where + "unknown type '" + type + "' (channel_delta, latent_attention)");
        }
        if (given(L, "mlp")) {
            const Json& mlp = need_obj(L, "mlp", where);
            const std::string kind = take_string(mlp, "kind", "dense");
            if (kind == "dense") {
                l.ffn = PartSpec("gated_mlp", obj({{"hidden_size", width}, {"intermediate_size", take_int(mlp, "ff")}, {"activation", std::string("relu")},
                                                   {"output_dtype", std::string("float32")},
                                                   {"names", name_map({{"gate", "gate"}, {"up", "up"}, {"down", "down"}})}}));
            } else if (kind == "moe") {
                const Json& router = need_obj(mlp, "router", where);
                l.ffn = PartSpec("routed_mlp", obj({{"hidden_size", width}, {"intermediate_size", take_int(need_obj(mlp, "expert", where), "ff")},
                                                    {"experts", take_int(router, "experts")}, {"top", take_int(router, "top")},
                                                    {"activation", std::string("silu")}, {"router_bias", true},
                                                    {"names", name_map({{"router", "router"}, {"router_bias", "router.b"}, {"expert", "e"},
                                                                        {"gate", "gate"}, {"up", "up"}, {"down", "down"}})}}));
            } else {
                throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not supported (dense, moe)");
            }
        }
        s.layers.push_back(l);
        i++;
    }
    // the order of execution: the looped layers run `times` times, every pass with cache entries of its own
    const long long n = (long long)s.layers.size();
    int cache = 0;
    auto run = [&](long long layer, bool reenter) { s.schedule.push_back(ScheduleEntry{(int)layer, cache++, true, reenter}); };
    if (!has_loop) {
        for (long long k = 0; k < n; k++) run(k, false);
    } else {
        for (long long k = 0; k < loop_start; k++) run(k, false);
        for (long long pass = 0; pass < loop_times; pass++)
            for (long long k = loop_start; k < loop_stop; k++) run(k, k == loop_start);
        for (long long k = loop_stop; k < n; k++) run(k, false);
        s.reentry = PartSpec("linear", obj({{"name", std::string("loop.")}, {"tensor", std::string("in")}, {"in_size", 2 * width}, {"out_size", width},
                                            {"output_dtype", std::string("float32")}}));
    }
    if (has_bigram)
        s.embedding = PartSpec("bigram_embedding", obj({{"name", std::string("")}, {"tensor", std::string("embed")}, {"bigram_tensor", std::string("bigram")},
                                                        {"vocab_size", vocab}, {"hidden_size", width}, {"buckets", buckets}, {"mul_prev", mul_prev},
                                                        {"mul_cur", mul_cur}}));
    else
        s.embedding = PartSpec("embedding", obj({{"name", std::string("embed")}, {"tensor", std::string("")}, {"vocab_size", vocab}, {"hidden_size", width}}));
    s.final_norm = PartSpec("rmsnorm", obj({{"name", std::string("final.norm")}, {"tensor", std::string("")}, {"size", width}, {"eps", norm_eps},
                                            {"float32_weight", true}}));
    s.head = PartSpec("lm_head", obj({{"name", std::string("head")}, {"tensor", std::string("")}, {"tied", true}, {"vocab_size", vocab},
                                      {"hidden_size", width}}));
    return s;
}

void register_vizosun_architecture() { register_architecture("Vizosun", &VizosunConfig::from_json, {"vizosun"}); }

}  // namespace illm
