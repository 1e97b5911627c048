#include "config/vokelix.h"

#include <cmath>

namespace illm {

static const Json& need_obj(const Json& d, const std::string& key, const std::string& where) {
    if (!d.is_object() || !d.has(key) || !d.at(key).is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return d.at(key);
}

std::unique_ptr<ArchConfig> VokelixConfig::from_json(const Json& d) {
    std::unique_ptr<VokelixConfig> c(new VokelixConfig);
    c->raw = d;
    c->width = take_int(d, "width");
    c->vocab = take_int(d, "vocab");
    c->max_positions = take_int(d, "max_positions", 131072);
    c->norm_eps = take_double(need_obj(d, "norm", ""), "eps", 1e-6);
    c->postln_alpha = take_double(d, "postln_alpha", 1.0);
    if (c->width <= 0 || c->vocab <= 0 || c->max_positions <= 0) throw ConfigError("config.json: width, vocab and max_positions must be positive");
    if (!(c->norm_eps > 0)) throw ConfigError("config.json: norm.eps must be positive");
    if (!d.has("layers") || !d.at("layers").is_array() || d.at("layers").size() == 0)
        throw ConfigError("config.json: 'layers' must be a list with at least one layer");
    c->model_spec();        // every layer is checked now, not at the first use
    return std::unique_ptr<ArchConfig>(c.release());
}

namespace {
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

ModelSpec VokelixConfig::model_spec() const {
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
        l.names = {{"mixer", "mix."}, {"ffn", "mlp."}, {"norm1", "norm1"}, {"norm2", "norm2"}};
        PartSpec norm("rmsnorm", obj({{"size", width}, {"eps", norm_eps}, {"weight_offset", 1.0}, {"residual_scale", postln_alpha},
                                      {"tensor", std::string("")}}));
        l.norms["norm1"] = norm;
        bool writes = true;
        int cache = (int)i;
        const long long heads = take_int(m, "heads"), dim = take_int(m, "dim"), vdim = take_int(m, "vdim");
        if (heads <= 0 || dim <= 0 || vdim <= 0) throw ConfigError("config.json: " + where + "heads, dim and vdim must be positive");
        if (type == "attention") {
            // softmax attention over grouped heads with biases on q, k, v, an RMS norm over the whole q and
            // the whole k projection, interleaved rotary positions with the stretched-frequency scaling, a
            // sink per head in the softmax denominator and a sigmoid gate per head on the output
            const long long kvh = take_int(m, "kv_heads");
            const Json& rot = need_obj(m, "rot", where);
            const long long rot_dims = take_int(rot, "dims");
            if (rot_dims <= 0 || rot_dims % 2 || rot_dims > dim) throw ConfigError("config.json: " + where + "rot.dims must be even and at most dim");
            Json pos = obj({{"head_dim", dim}, {"rot_dim", rot_dims}, {"theta", take_double(rot, "base", 10000.0)}, {"max_positions", max_positions}});
            if (rot.has("scaling") && rot.at("scaling").is_object()) pos.set("scaling", rot.at("scaling"));
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"n_kv_heads", kvh}, {"head_dim", dim}, {"v_head_dim", vdim},
                          {"scale", take_double(m, "scale", 1.0 / std::sqrt((double)dim))}, {"qkv_bias", true}, {"qk_norm", std::string("projection")},
                          {"norm_eps", norm_eps}, {"sink", true}, {"out_gate", std::string("head_sigmoid")}, {"output_dtype", std::string("float32")},
                          {"position", PartSpec("rope_pairs", pos).to_json()},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"q_bias", "q.b"}, {"k_bias", "k.b"}, {"v_bias", "v.b"},
                                              {"q_norm", "q.norm"}, {"k_norm", "k.norm"}, {"sink", "sink"}, {"gate", "g"}})}});
            if (m.has("kv_from") && !m.at("kv_from").is_null()) {
                // the layer attends to the keys and values that an earlier attention layer put into its cache entry
                const long long j = take_int(m, "kv_from");
                if (j < 0 || j >= (long long)i) throw ConfigError("config.json: " + where + "kv_from must name an earlier layer");
                const LayerSpec& src = s.layers[(size_t)j];
                if (src.mixer.kind != "attention" || !src.mixer.get_bool("own_kv", true) || src.mixer.get_int("n_kv_heads") != kvh ||
                    src.mixer.get_int("head_dim") != dim || src.mixer.get_int("v_head_dim") != vdim)
                    throw ConfigError("config.json: " + where + "kv_from must name an attention layer with keys and values of its own and the same head count and sizes");
                p.set("own_kv", false);
                writes = false;
                cache = (int)j;
            }
            l.mixer = PartSpec("attention", p);
        } else if (type == "lightning" || type == "retention") {
            if (!m.has("decay") || !m.at("decay").is_array() || (long long)m.at("decay").size() != heads)
                throw ConfigError("config.json: " + where + "'decay' must list one number per head");
            Json p = obj({{"hidden_size", width}, {"n_heads", heads}, {"head_dim", dim}, {"v_head_dim", vdim}, {"decay", m.at("decay")},
                          {"norm_eps", norm_eps}, {"output_dtype", std::string("float32")},
                          {"names", name_map({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"gate", "g"}, {"o", "o"}, {"norm", "norm"}})}});
            if (type == "lightning") {
                // silu on q, k and v; one weighted norm over all heads; a sigmoid gate
                p.set("qk_activation", std::string("silu"));
                p.set("v_activation", std::string("silu"));
                p.set("out_norm", std::string("joint"));
                p.set("gate_activation", std::string("sigmoid"));
            } else {
                // rotate-half positions on q and k, k scaled by dim^(-1/2); a norm without weight per head; a silu gate
                const Json& rot = need_obj(m, "rot", where);
                const long long rot_dims = take_int(rot, "dims");
                if (rot_dims <= 0 || rot_dims % 2 || rot_dims > dim) throw ConfigError("config.json: " + where + "rot.dims must be even and at most dim");
                p.set("position", PartSpec("rope_half", obj({{"head_dim", dim}, {"rot_dim", rot_dims}, {"theta", take_double(rot, "base", 10000.0)},
                                                             {"max_positions", max_positions}})).to_json());
                p.set("k_scale", 1.0 / std::sqrt((double)dim));
                p.set("out_norm", std::string("per_head"));
                p.set("gate_activation", std::string("silu"));
            }
            l.mixer = PartSpec("decay_linear_attention", p);
        } else {
            throw ConfigError("config.json: " + where + "unknown type '" + type + "' (attention, lightning, retention)");
        }
        if (L.has("mlp") && !L.at("mlp").is_null()) {
            const Json& mlp = need_obj(L, "mlp", where);
            const std::string kind = take_string(mlp, "kind", "dense");
            if (kind != "dense") throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not supported (dense)");
            l.block = "postnorm";
            l.ffn = PartSpec("gated_mlp", obj({{"hidden_size", width}, {"intermediate_size", take_int(mlp, "ff")}, {"activation", std::string("silu")},
                                               {"output_dtype", std::string("float32")},
                                               {"names", name_map({{"gate", "gate"}, {"up", "up"}, {"down", "down"}})}}));
            l.norms["norm2"] = norm;
        } else {
            // no feed-forward: the layer ends after norm1; should a weight file hold a norm2 for it all the same, it is applied
            // to the scaled stream alone (the norm is declared optional)
            l.block = "postnorm_mixer";
            PartSpec norm2 = norm;
            norm2.params.set("optional", true);
            l.norms["norm2"] = norm2;
        }
        s.layers.push_back(l);
        s.schedule.push_back(ScheduleEntry{(int)i, cache, writes});
        i++;
    }
    s.embedding = PartSpec("embedding", obj({{"name", std::string("embed")}, {"tensor", std::string("")}, {"vocab_size", vocab}, {"hidden_size", width}}));
    s.final_norm = PartSpec("rmsnorm", obj({{"name", std::string("final.norm")}, {"tensor", std::string("")}, {"size", width}, {"eps", norm_eps},
                                            {"weight_offset", 1.0}}));
    s.head = PartSpec("lm_head", obj({{"name", std::string("head")}, {"tensor", std::string("")}, {"tied", false}, {"vocab_size", vocab},
                                      {"hidden_size", width}}));
    return s;
}

void register_vokelix_architecture() { register_architecture("Vokelix", &VokelixConfig::from_json, {"vokelix"}); }

}  // namespace illm
