// The Zuzelorn decoder's typed configuration (see zuzelorn.cpp).
#pragma once

#include <string>
#include <vector>

#include "registry.h"

namespace jb {

struct ZuzelornConfig : ArchConfig {
    struct Layer {
        std::string type;                 // which mixer: "attention"
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        double scale = 0;
        long long kv_from = -1;           // the layer whose keys and values this one reads; -1: its own
        bool has_mlp = false;
        std::string mlp_kind;             // "dense"
        long long ff = 0;
    };
    long long vocab = 0, width = 0, max_positions = 0;
    double norm_eps = 0, logit_scale = 1.0;
    std::vector<Layer> layers;

    static ZuzelornConfig from_json(const Json &config_json);
    void validate() const;

    std::string architecture() const override { return "Zuzelorn"; }
    Json to_json() const override;
    ModelSpec to_model_spec() const override;
};

void register_zuzelorn();

}  // namespace jb
