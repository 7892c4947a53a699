// Typed configuration of the Zuzelorn decoder, read from its config.json.
//
// The file names the design ("architecture": "Zuzelorn"), the sizes (vocab, width,
// max_positions), the constants (norm.eps, logit_scale) and a list of layers; each
// layer gives its mixer's type and sizes (heads, kv_heads, dim, vdim, scale, and
// kv_from for a layer that reads another layer's keys and values) and its
// feed-forward (kind, ff) or null for none.  Every size and constant comes from
// the file; what the design fixes is written here: a learned position vector is
// added to each embedding row, every norm is a Dynamic Tanh, each sublayer has a
// norm before and after it and a sigmoid gate on its result, the attention has
// biases, a factor per head, a sink per head and no rotation, the feed-forward's
// activation is PolyNorm, and the logits are scaled.
//
// Tensor names: embed, pos, head, final.norm; layer i below "l<i>": norm1, norm1b,
// norm2, norm2b (each with .b and .alpha), mix.{q,k,v,o} (each with .b), mix.temp,
// mix.sink, mlp.{up,down,act}, rg1, rg2 (each with .b).
#include "zuzelorn.h"

namespace jb {

static long long need_int(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number() || !v.whole())
        config_error("config.json: " + where + key + " must be a whole number, got " + v.dump());
    return v.as_int();
}

static double need_num(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number())
        config_error("config.json: " + where + key + " must be a number, got " + v.dump());
    return v.as_double();
}

ZuzelornConfig ZuzelornConfig::from_json(const Json &d) {
    ZuzelornConfig c;
    c.vocab = need_int(d, "vocab", "");
    c.width = need_int(d, "width", "");
    c.max_positions = need_int(d, "max_positions", "");
    if (!d.get("norm").is_object()) config_error("config.json: norm must be an object with eps");
    c.norm_eps = need_num(d.get("norm"), "eps", "norm.");
    c.logit_scale = d.get("logit_scale").is_null() ? 1.0 : need_num(d, "logit_scale", "");
    const Json &ls = d.get("layers");
    if (!ls.is_array() || ls.size() == 0) config_error("config.json: layers must be a list of layers");
    for (size_t i = 0; i < ls.size(); i++) {
        const Json &l = ls[i];
        std::string where = fmt("layers[%zu].", i);
        if (!l.is_object() || !l.get("type").is_string() || !l.get("mixer").is_object())
            config_error("config.json: " + where + " needs a type and a mixer");
        Layer y;
        y.type = l.get("type").as_string();
        if (y.type != "attention")
            config_error("config.json: " + where + "type '" + y.type + "': this design's mixer is 'attention'");
        const Json &m = l.get("mixer");
        std::string mw = where + "mixer.";
        y.heads = need_int(m, "heads", mw);
        y.kv_heads = need_int(m, "kv_heads", mw);
        y.dim = need_int(m, "dim", mw);
        y.vdim = m.get("vdim").is_null() ? y.dim : need_int(m, "vdim", mw);
        y.scale = need_num(m, "scale", mw);
        y.kv_from = m.get("kv_from").is_null() ? -1 : need_int(m, "kv_from", mw);
        const Json &f = l.get("mlp");
        if (!f.is_null()) {
            if (!f.is_object() || !f.get("kind").is_string())
                config_error("config.json: " + where + "mlp must be null or an object with kind and ff");
            y.has_mlp = true;
            y.mlp_kind = f.get("kind").as_string();
            if (y.mlp_kind != "dense")
                config_error("config.json: " + where + "mlp.kind '" + y.mlp_kind + "': this design's is 'dense'");
            y.ff = need_int(f, "ff", where + "mlp.");
        }
        c.layers.push_back(y);
    }
    c.validate();
    return c;
}

void ZuzelornConfig::validate() const {
    if (vocab <= 0 || width <= 0 || max_positions <= 0)
        config_error("config.json: vocab, width and max_positions must be positive");
    if (layers.empty() || layers.size() > 100000) config_error("config.json: layers must not be empty");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        std::string where = fmt("config.json: layers[%zu]: ", i);
        if (y.heads <= 0 || y.kv_heads <= 0 || y.dim <= 0 || y.vdim <= 0)
            config_error(where + "heads, kv_heads, dim and vdim must be positive");
        if (y.heads % y.kv_heads) config_error(where + "heads must be a multiple of kv_heads");
        if (y.dim > 512 || y.vdim > 512) config_error(where + "the attention kernels take head sizes up to 512");
        if (y.has_mlp && y.ff <= 0) config_error(where + "mlp.ff must be positive");
        if (y.kv_from >= 0) {
            if (y.kv_from >= (long long)i) config_error(where + "kv_from must name an earlier layer");
            const Layer &src = layers[(size_t)y.kv_from];
            if (src.kv_from >= 0) config_error(where + "kv_from names a layer that has no keys and values of its own");
            if (src.kv_heads != y.kv_heads || src.dim != y.dim || src.vdim != y.vdim)
                config_error(where + "kv_from names a layer with other kv_heads, dim or vdim");
        }
    }
}

Json ZuzelornConfig::to_json() const {
    Json d = Json::object();
    d.set("architecture", "Zuzelorn");
    Json ls = Json::array();
    for (auto &y : layers) {
        Json l = Json::object(), m = Json::object();
        m.set("dim", y.dim);
        m.set("heads", y.heads);
        if (y.kv_from >= 0) m.set("kv_from", y.kv_from);
        m.set("kv_heads", y.kv_heads);
        m.set("scale", y.scale);
        m.set("vdim", y.vdim);
        l.set("mixer", m);
        if (y.has_mlp) {
            Json f = Json::object();
            f.set("ff", y.ff);
            f.set("kind", y.mlp_kind);
            l.set("mlp", f);
        } else {
            l.set("mlp", Json());
        }
        l.set("type", y.type);
        ls.push(l);
    }
    d.set("layers", ls);
    d.set("logit_scale", logit_scale);
    d.set("max_positions", max_positions);
    Json n = Json::object();
    n.set("eps", norm_eps);
    d.set("norm", n);
    d.set("vocab", vocab);
    d.set("width", width);
    return d;
}

ModelSpec ZuzelornConfig::to_model_spec() const {
    // every norm: Dynamic Tanh over the width; the weight is the tensor named as the norm
    PartSpec norm{"dynamic_tanh", Json::object()};
    norm.params.set("size", width);
    {
        Json nm = Json::object();
        nm.set("weight", "");
        nm.set("bias", "b");
        nm.set("alpha", "alpha");
        norm.params.set("names", nm);
    }
    ModelSpec s;
    s.architecture = "Zuzelorn";
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = max_positions;
    s.embedding_name = "embed";
    s.position_table_name = "pos";
    s.head_name = "head";
    s.final_norm_name = "final.norm";
    s.final_norm = norm;
    s.tie_embeddings = false;
    s.logit_scale = logit_scale;
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        PartSpec mixer{"sink_attention", Json::object()};
        mixer.params.set("hidden_size", width);
        mixer.params.set("num_heads", y.heads);
        mixer.params.set("num_kv_heads", y.kv_heads);
        mixer.params.set("head_dim", y.dim);
        mixer.params.set("v_head_dim", y.vdim);
        mixer.params.set("scale", y.scale);
        mixer.params.set("window", 0);
        mixer.params.set("bias", true);
        mixer.params.set("head_scale", true);
        mixer.params.set("sink", true);
        mixer.params.set("own_kv", y.kv_from < 0);
        {
            Json nm = Json::object();
            nm.set("q", "q");
            nm.set("k", "k");
            nm.set("v", "v");
            nm.set("o", "o");
            nm.set("bias", ".b");
            nm.set("head_scale", "temp");
            nm.set("sink", "sink");
            mixer.params.set("names", nm);
        }
        LayerSpec l;
        l.block = "sandwich";
        l.prefix = fmt("l%zu", i);
        l.mixer = mixer;
        l.mixer_name = "mix";
        l.mixer_norm = norm;
        l.mixer_norm_name = "norm1";
        l.post_mixer_norm = norm;
        l.post_mixer_norm_name = "norm1b";
        l.block_params.set("hidden_size", width);
        l.block_params.set("mixer_gate", "rg1");
        l.block_params.set("gate_bias", ".b");
        if (y.has_mlp) {
            PartSpec ffn{"polynorm", Json::object()};
            ffn.params.set("hidden_size", width);
            ffn.params.set("intermediate_size", y.ff);
            ffn.params.set("eps", norm_eps);
            Json nm = Json::object();
            nm.set("up", "up");
            nm.set("down", "down");
            nm.set("coefficients", "act");
            ffn.params.set("names", nm);
            l.feed_forward = ffn;
            l.ffn_name = "mlp";
            l.ffn_norm = norm;
            l.ffn_norm_name = "norm2";
            l.post_ffn_norm = norm;
            l.post_ffn_norm_name = "norm2b";
            l.block_params.set("ffn_gate", "rg2");
        } else {
            // a layer without a feed-forward has none of its surroundings either; a file
            // that holds them all the same is read without complaint
            Json unused = Json::array();
            auto vec = [&](const std::string &name, bool scalar) {
                Json u = Json::object(), shape = Json::array();
                if (!scalar) shape.push(width);
                u.set("name", name);
                u.set("shape", shape);
                unused.push(u);
            };
            for (const char *nn : {"norm2", "norm2b"}) {
                vec(nn, false);
                vec(std::string(nn) + ".b", false);
                vec(std::string(nn) + ".alpha", true);
            }
            vec("rg2.b", false);
            Json u = Json::object(), shape = Json::array();
            shape.push(width);
            shape.push(width);
            u.set("name", "rg2");
            u.set("shape", shape);
            unused.push(u);
            l.block_params.set("unused", unused);
        }
        s.layers.push_back(l);
        // a layer that reads another's keys and values: that layer's place in the cache
        s.run_order.push_back(RunEntry{(int)i, (int)y.kv_from});
    }
    s.validate();
    return s;
}

void register_zuzelorn() {
    register_architecture("Zuzelorn", "zuzelorn", [](const Json &d) {
        return std::unique_ptr<ArchConfig>(new ZuzelornConfig(ZuzelornConfig::from_json(d)));
    });
}

}  // namespace jb
