// Typed configuration of the Vokelix decoder, read from its config.json keys.
//
// A Vokelix model lists its layers one by one: `layers[i]` has `type` ("attention", "lightning" or
// "retention": which mixer), `mixer` (the mixer's sizes and constants) and `mlp` ({"kind": "dense",
// "ff": n} or null for a layer without a feed-forward).  Beside the list there are `width`, `vocab`,
// `norm.eps` and `postln_alpha`, and optionally `max_positions` (the longest sequence a rotation
// table is made for; 131072 if not given).  Every layer is a norm-after-the-sum block; what the three
// mixers are is said where they are mapped to parts (config/vokelix.cpp).
#pragma once
#include "config/config.h"

namespace illm {

struct VokelixConfig : ArchConfig {
    Json raw;                    // the config.json object as it was read (to_json gives it back)
    long long width = 0, vocab = 0, max_positions = 131072;
    double norm_eps = 1e-6, postln_alpha = 1.0;

    static std::unique_ptr<ArchConfig> from_json(const Json& d);
    std::string architecture() const override { return "Vokelix"; }
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
};

}  // namespace illm
