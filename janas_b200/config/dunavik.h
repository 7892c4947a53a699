// The Dunavik decoder's typed configuration (see dunavik.cpp).
#pragma once

#include <string>
#include <vector>

#include "registry.h"

namespace jb {

struct DunavikConfig : ArchConfig {
    struct Layer {
        std::string type;                 // which mixer: "latent_attention" or "attention"
        long long heads = 0, dim = 0, vdim = 0;
        double scale = 0;
        // latent_attention
        long long kv_rank = 0, q_rank = 0, rot_dim = 0, rot_dims = 0;
        double rot_base = 0;
        // attention
        long long kv_heads = 0;
        long long window = 0;             // mask.size; 0: every earlier position is seen
        double softcap = 0;               // 0: none
        double q_temp_coef = 0;
        long long q_temp_every = 0;       // 0: no query temperature
        bool has_mlp = false;
        std::string mlp_kind;             // "dense"
        long long ff = 0;
    };
    long long vocab = 0, width = 0;
    double norm_eps = 0, residual_mult = 1.0;
    long long loop_start = 0, loop_stop = 0, loop_times = 1;      // times 1: every layer runs once
    std::vector<Layer> layers;

    static DunavikConfig from_json(const Json &config_json);
    void validate() const;
    // the layers in the order they run: (layer, whether the embedding output is added before it)
    std::vector<std::pair<int, bool>> order() const;

    std::string architecture() const override { return "Dunavik"; }
    Json to_json() const override;
    ModelSpec to_model_spec() const override;
};

void register_dunavik();

}  // namespace jb
