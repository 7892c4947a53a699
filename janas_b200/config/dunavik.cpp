// Typed configuration of the Dunavik decoder, read from its config.json.
//
// The file names the design ("architecture": "Dunavik"), the sizes (vocab, width),
// the constants (norm.eps, residual_mult), a list of layers and a loop.  Each layer
// gives its mixer's type and sizes and its feed-forward (kind, ff) or null for none:
//
//   type "latent_attention": heads, dim (plain query/key values per head), rot_dim
//       (rotated ones), vdim, kv_rank, q_rank, scale, rot {base, dims}
//   type "attention": heads, kv_heads, dim, vdim, scale, and optionally softcap,
//       mask {size} (a sliding window) and q_temp {coef, every}
//
// loop {start, stop, times}: layers start .. stop-1 run `times` times in a row with
// the same weights; every pass is a run-order entry of its own per layer (its own
// place in the cache), and every pass but the first begins by adding the embedding
// output to the residual stream.
//
// What the design fixes is written here: the embedding rows go through a layer norm;
// every norm is a layer norm with weight and bias; a layer has one norm, mixer and
// feed-forward read its output side by side and their sum joins the residual stream
// times residual_mult; the attention mixer has no rotation, takes slope * distance
// off its scores with slope 2^(-8 (head + 1) / heads), after the cap; the latent
// mixer rotates neighbouring pairs and gates its heads' outputs with a sigmoid; the
// feed-forward's activation is the square of relu.
//
// Tensor names: embed, embed.norm (+ .b), head, final.norm (+ .b); layer i below
// "l<i>": norm1 (+ .b), mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o} or
// mix.{q, k, v, o}, mlp.{up, down}.
#include "dunavik.h"

namespace jb {

namespace {

long long need_int(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number() || !v.whole())
        config_error("config.json: " + where + key + " must be a whole number, got " + v.dump());
    return v.as_int();
}

double need_num(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number())
        config_error("config.json: " + where + key + " must be a number, got " + v.dump());
    return v.as_double();
}

}  // namespace

DunavikConfig DunavikConfig::from_json(const Json &d) {
    DunavikConfig c;
    c.vocab = need_int(d, "vocab", "");
    c.width = need_int(d, "width", "");
    if (!d.get("norm").is_object()) config_error("config.json: norm must be an object with eps");
    c.norm_eps = need_num(d.get("norm"), "eps", "norm.");
    c.residual_mult = d.get("residual_mult").is_null() ? 1.0 : need_num(d, "residual_mult", "");
    const Json &ls = d.get("layers");
    if (!ls.is_array() || ls.size() == 0) config_error("config.json: layers must be a list of layers");
    for (size_t i = 0; i < ls.size(); i++) {
        const Json &l = ls[i];
        std::string where = fmt("layers[%zu].", i);
        if (!l.is_object() || !l.get("type").is_string() || !l.get("mixer").is_object())
            config_error("config.json: " + where + " needs a type and a mixer");
        Layer y;
        y.type = l.get("type").as_string();
        const Json &m = l.get("mixer");
        std::string mw = where + "mixer.";
        y.heads = need_int(m, "heads", mw);
        y.dim = need_int(m, "dim", mw);
        y.vdim = m.get("vdim").is_null() ? y.dim : need_int(m, "vdim", mw);
        y.scale = need_num(m, "scale", mw);
        if (y.type == "latent_attention") {
            y.kv_rank = need_int(m, "kv_rank", mw);
            y.q_rank = need_int(m, "q_rank", mw);
            y.rot_dim = need_int(m, "rot_dim", mw);
            if (!m.get("rot").is_object()) config_error("config.json: " + mw + "rot must be an object with base and dims");
            y.rot_base = need_num(m.get("rot"), "base", mw + "rot.");
            y.rot_dims = need_int(m.get("rot"), "dims", mw + "rot.");
        } else if (y.type == "attention") {
            y.kv_heads = m.get("kv_heads").is_null() ? y.heads : need_int(m, "kv_heads", mw);
            if (!m.get("mask").is_null()) {
                if (!m.get("mask").is_object()) config_error("config.json: " + mw + "mask must be an object with size");
                y.window = need_int(m.get("mask"), "size", mw + "mask.");
                if (y.window <= 0) config_error("config.json: " + mw + "mask.size must be positive");
            }
            if (!m.get("softcap").is_null()) y.softcap = need_num(m, "softcap", mw);
            if (!m.get("q_temp").is_null()) {
                if (!m.get("q_temp").is_object())
                    config_error("config.json: " + mw + "q_temp must be an object with coef and every");
                y.q_temp_coef = need_num(m.get("q_temp"), "coef", mw + "q_temp.");
                y.q_temp_every = need_int(m.get("q_temp"), "every", mw + "q_temp.");
                if (y.q_temp_every <= 0) config_error("config.json: " + mw + "q_temp.every must be positive");
            }
        } else {
            config_error("config.json: " + where + "type '" + y.type +
                         "': this design's mixers are 'latent_attention' and 'attention'");
        }
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
    const Json &lp = d.get("loop");
    if (!lp.is_null()) {
        if (!lp.is_object()) config_error("config.json: loop must be null or an object with start, stop and times");
        c.loop_start = need_int(lp, "start", "loop.");
        c.loop_stop = need_int(lp, "stop", "loop.");
        c.loop_times = need_int(lp, "times", "loop.");
    }
    c.validate();
    return c;
}

void DunavikConfig::validate() const {
    if (vocab <= 0 || width <= 0) config_error("config.json: vocab and width must be positive");
    if (layers.empty() || layers.size() > 100000) config_error("config.json: layers must not be empty");
    long long n = (long long)layers.size();
    if (loop_start < 0 || loop_stop < loop_start || loop_stop > n || loop_times < 1 || loop_times > 100000)
        config_error("config.json: loop needs 0 <= start <= stop <= the number of layers and times >= 1");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        std::string where = fmt("config.json: layers[%zu]: ", i);
        if (y.heads <= 0 || y.dim <= 0 || y.vdim <= 0) config_error(where + "heads, dim and vdim must be positive");
        if (y.has_mlp && y.ff <= 0) config_error(where + "mlp.ff must be positive");
        if (y.type == "latent_attention") {
            if (y.kv_rank <= 0 || y.q_rank <= 0 || y.rot_dim < 0)
                config_error(where + "kv_rank and q_rank must be positive, rot_dim not negative");
            if (y.rot_dims < 0 || y.rot_dims % 2 || y.rot_dims > y.rot_dim)
                config_error(where + "rot.dims must be even and at most rot_dim");
            if (y.rot_dims > 0 && y.rot_base <= 0) config_error(where + "rot.base must be positive");
            if (y.kv_rank + y.rot_dim > 512)
                config_error(where + "kv_rank + rot_dim is above 512, the longest row the attention kernels take");
        } else {
            if (y.kv_heads <= 0 || y.heads % y.kv_heads) config_error(where + "heads must be a multiple of kv_heads");
            if (y.dim > 512 || y.vdim > 512) config_error(where + "the attention kernels take head sizes up to 512");
            if (y.softcap < 0) config_error(where + "softcap must not be negative");
        }
    }
}

std::vector<std::pair<int, bool>> DunavikConfig::order() const {
    std::vector<std::pair<int, bool>> out;
    int n = (int)layers.size();
    for (int i = 0; i < (int)loop_start; i++) out.push_back({i, false});
    for (long long pass = 0; pass < loop_times; pass++)
        for (int i = (int)loop_start; i < (int)loop_stop; i++) out.push_back({i, pass > 0 && i == (int)loop_start});
    for (int i = (int)loop_stop; i < n; i++) out.push_back({i, false});
    return out;
}

Json DunavikConfig::to_json() const {
    Json d = Json::object();
    d.set("architecture", "Dunavik");
    Json ls = Json::array();
    for (auto &y : layers) {
        Json l = Json::object(), m = Json::object();
        m.set("dim", y.dim);
        m.set("heads", y.heads);
        if (y.type == "latent_attention") {
            m.set("kv_rank", y.kv_rank);
            m.set("q_rank", y.q_rank);
            Json r = Json::object();
            r.set("base", y.rot_base);
            r.set("dims", y.rot_dims);
            m.set("rot", r);
            m.set("rot_dim", y.rot_dim);
        } else {
            m.set("kv_heads", y.kv_heads);
            if (y.window > 0) {
                Json w = Json::object();
                w.set("size", y.window);
                m.set("mask", w);
            }
            if (y.q_temp_every > 0) {
                Json q = Json::object();
                q.set("coef", y.q_temp_coef);
                q.set("every", y.q_temp_every);
                m.set("q_temp", q);
            }
            if (y.softcap > 0) m.set("softcap", y.softcap);
        }
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
    Json lp = Json::object();
    lp.set("start", loop_start);
    lp.set("stop", loop_stop);
    lp.set("times", loop_times);
    d.set("loop", lp);
    Json n = Json::object();
    n.set("eps", norm_eps);
    d.set("norm", n);
    d.set("residual_mult", residual_mult);
    d.set("vocab", vocab);
    d.set("width", width);
    return d;
}

ModelSpec DunavikConfig::to_model_spec() const {
    // every norm: a layer norm over the width; the weight is the tensor named as the
    // norm, its bias has ".b" added
    PartSpec norm{"layernorm", Json::object()};
    norm.params.set("size", width);
    norm.params.set("eps", norm_eps);
    {
        Json nm = Json::object();
        nm.set("weight", "");
        nm.set("bias", "b");
        norm.params.set("names", nm);
    }
    // the design gives no limit on positions: the cache's size is the limit
    const long long positions = 1ll << 30;
    ModelSpec s;
    s.architecture = "Dunavik";
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = positions;
    s.embedding_name = "embed";
    s.embedding_norm = norm;
    s.embedding_norm_name = "embed.norm";
    s.head_name = "head";
    s.final_norm_name = "final.norm";
    s.final_norm = norm;
    s.tie_embeddings = false;
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        PartSpec mixer;
        if (y.type == "latent_attention") {
            mixer.kind = "latent_attention";
            mixer.params.set("hidden_size", width);
            mixer.params.set("num_heads", y.heads);
            mixer.params.set("head_dim", y.dim);
            mixer.params.set("rot_dim", y.rot_dim);
            mixer.params.set("v_head_dim", y.vdim);
            mixer.params.set("kv_rank", y.kv_rank);
            mixer.params.set("q_rank", y.q_rank);
            mixer.params.set("scale", y.scale);
            mixer.params.set("eps", norm_eps);
            mixer.params.set("gate", true);
            PartSpec pos;
            if (y.rot_dims > 0) {
                pos.kind = "rope_pairs";
                pos.params.set("rotary_dim", y.rot_dims);
                pos.params.set("theta", y.rot_base);
                pos.params.set("max_positions", positions);
            } else {
                pos.kind = "none";
            }
            mixer.params.set("position", pos.to_json());
            Json nm = Json::object();
            nm.set("dq", "dq");
            nm.set("dq_norm", "dq.norm");
            nm.set("uq", "uq");
            nm.set("dkv", "dkv");
            nm.set("dkv_norm", "dkv.norm");
            nm.set("uk", "uk");
            nm.set("uv", "uv");
            nm.set("gate", "g");
            nm.set("o", "o");
            mixer.params.set("names", nm);
        } else {
            mixer.kind = "sink_attention";
            mixer.params.set("hidden_size", width);
            mixer.params.set("num_heads", y.heads);
            mixer.params.set("num_kv_heads", y.kv_heads);
            mixer.params.set("head_dim", y.dim);
            mixer.params.set("v_head_dim", y.vdim);
            mixer.params.set("scale", y.scale);
            mixer.params.set("window", y.window);
            if (y.softcap > 0) mixer.params.set("softcap", y.softcap);
            mixer.params.set("distance_slope_exponent", 8.0);
            if (y.q_temp_every > 0) {
                mixer.params.set("q_temp_coef", y.q_temp_coef);
                mixer.params.set("q_temp_every", y.q_temp_every);
            }
            mixer.params.set("bias", false);
            mixer.params.set("head_scale", false);
            mixer.params.set("sink", false);
            mixer.params.set("own_kv", true);
            Json nm = Json::object();
            nm.set("q", "q");
            nm.set("k", "k");
            nm.set("v", "v");
            nm.set("o", "o");
            mixer.params.set("names", nm);
        }
        LayerSpec l;
        l.block = "parallel";
        l.prefix = fmt("l%zu", i);
        l.mixer = mixer;
        l.mixer_name = "mix";
        l.mixer_norm = norm;
        l.mixer_norm_name = "norm1";
        l.block_params.set("residual_mult", residual_mult);
        if (y.has_mlp) {
            PartSpec ffn{"dense", Json::object()};
            ffn.params.set("hidden_size", width);
            ffn.params.set("intermediate_size", y.ff);
            ffn.params.set("activation", "relu2");
            Json nm = Json::object();
            nm.set("up", "up");
            nm.set("down", "down");
            ffn.params.set("names", nm);
            l.feed_forward = ffn;
            l.ffn_name = "mlp";
        }
        s.layers.push_back(l);
    }
    for (auto &e : order()) {
        RunEntry r;
        r.layer = e.first;
        r.add_embedding = e.second;
        s.run_order.push_back(r);
    }
    s.validate();
    return s;
}

void register_dunavik() {
    register_architecture("Dunavik", "dunavik", [](const Json &d) {
        return std::unique_ptr<ArchConfig>(new DunavikConfig(DunavikConfig::from_json(d)));
    });
}

}  // namespace jb
