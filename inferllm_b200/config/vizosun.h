// Typed configuration of the Vizosun decoder, read from its config.json keys.
//
// A Vizosun model lists its layers one by one: `layers[i]` has `type` ("channel_delta" or "latent_attention":
// which mixer), `mixer` (the mixer's sizes and constants) and `mlp` ({"kind": "dense", "ff": n}, {"kind": "moe",
// "expert": {"ff": n}, "router": {"experts": E, "top": k}}, or null for a layer without a feed-forward).  Beside the
// list: `width`, `vocab`, `norm.eps`, optionally `embedding.bigram` {buckets, mul_prev, mul_cur} (a hashed bigram
// table added to the token embedding), optionally `loop` {start, stop, times} (layers start .. stop - 1 run `times`
// times in a row with the same weights and a cache entry per pass, each pass entered through the map `loop.in` of
// the stream joined with the embedding output), and optionally `max_positions` (the longest sequence; 131072 if not
// given).  Every layer is a parallel block: one norm whose output both sublayers read.  The output matrix is the
// embedding table.  What the two mixers are is said where they are mapped to parts (config/vizosun.cpp).
#pragma once
#include "config/config.h"

namespace illm {

struct VizosunConfig : ArchConfig {
    Json raw;                    // the config.json object as it was read (to_json gives it back)
    long long width = 0, vocab = 0, max_positions = 131072;
    double norm_eps = 1e-6;
    bool has_bigram = false, has_loop = false;
    long long buckets = 0, mul_prev = 0, mul_cur = 0;
    long long loop_start = 0, loop_stop = 0, loop_times = 1;

    static std::unique_ptr<ArchConfig> from_json(const Json& d);
    std::string architecture() const override { return "Vizosun"; }
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
};

}  // namespace illm
