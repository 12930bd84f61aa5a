// zelunex.cpp — the Zelunex family: a decoder of PARALLEL blocks (one RMS norm feeds the mixer and the feed-forward; both
// branches carry a per-channel layer scale and the sum enters the residual through a constant multiplier) whose mixer is
// windowed attention without positional rotation (kept first tokens, soft-capped scores, RMS norm over the whole query / key
// projection) and whose feed-forward is a tanh-GELU gated unit.  Layers may share another layer's tensors while keeping a
// cache of their own.  Everything that varies between models of the family is read from config.json.
#include "model_registry.h"
#include <algorithm>

namespace nt { namespace b200 {

namespace {

bool need_int(const Json& o, const char* key, int& out, std::string& err, const std::string& where) {
    const Json& v = o.at(key);
    if (!v.is_number()) { err = where + ": \"" + key + "\" is missing or not a number"; return false; }
    out = (int)v.int_or(0);
    return true;
}
bool need_float(const Json& o, const char* key, float& out, std::string& err, const std::string& where) {
    const Json& v = o.at(key);
    if (!v.is_number()) { err = where + ": \"" + key + "\" is missing or not a number"; return false; }
    out = (float)v.number_or(0.0);
    return true;
}

bool config_from_json(const Json& root, ModelConfig& cfg, std::string& err) {
    if (!need_int(root, "vocab", cfg.vocab_size, err, "config") || !need_int(root, "width", cfg.hidden_size, err, "config")) return false;
    if (!need_float(root.at("norm"), "eps", cfg.norm_eps, err, "config.norm")) return false;
    if (!need_float(root, "residual_mult", cfg.residual_mult, err, "config")) return false;
    const Json& layers = root.at("layers");
    if (!layers.is_array() || layers.arr.empty()) { err = "config: \"layers\" must be a non-empty list"; return false; }
    cfg.n_layers = (int)layers.arr.size();
    cfg.model_name = "zelunex";
    cfg.bos_token_id = -1; cfg.eos_token_id = -1;
    for (size_t i = 0; i < layers.arr.size(); i++) {
        const Json& e = layers.arr[i];
        const std::string where = "config.layers[" + std::to_string(i) + "]";
        LayerSpec L;
        const std::string type = e.at("type").string_or("");
        if (type != "attention") { err = where + ": mixer type \"" + type + "\" is not part of this family"; return false; }
        L.mixer = MixerKind::ATTN_WINDOW;
        L.form = BlockForm::PARALLEL;
        L.qk_norm = QKNorm::WHOLE;
        L.layer_scale = true;
        L.act = GluAct::GELU_TANH;
        const Json& m = e.at("mixer");
        if (!m.is_object()) { err = where + ": \"mixer\" is missing"; return false; }
        if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "kv_heads", L.kv_heads, err, where) || !need_int(m, "dim", L.dim, err, where) ||
            !need_int(m, "vdim", L.vdim, err, where) || !need_float(m, "scale", L.scale, err, where) || !need_float(m, "softcap", L.softcap, err, where))
            return false;
        const Json& mask = m.at("mask");
        if (!need_int(mask, "size", L.window, err, where + ".mask") || !need_int(mask, "keep_first", L.keep_first, err, where + ".mask")) return false;
        if (L.heads <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads || L.dim <= 0 || L.vdim <= 0 || L.window <= 0 || L.keep_first < 0) {
            err = where + ": invalid mixer sizes"; return false;
        }
        const Json& mlp = e.at("mlp");
        if (mlp.is_null()) L.ff = 0;
        else {
            const std::string kind = mlp.at("kind").string_or("");
            if (kind != "dense") { err = where + ": feed-forward kind \"" + kind + "\" is not part of this family"; return false; }
            if (!need_int(mlp, "ff", L.ff, err, where + ".mlp") || L.ff <= 0) { if (err.empty()) err = where + ": invalid ff"; return false; }
        }
        if (e.has("weights_of")) {
            L.weights_of = (int)e.at("weights_of").int_or(-1);
            if (L.weights_of < 0 || L.weights_of >= (int)i || cfg.layers[(size_t)L.weights_of].weights_of >= 0) {
                err = where + ": \"weights_of\" must name an earlier layer that owns its tensors"; return false;
            }
        }
        cfg.layers.push_back(L);
    }
    // the Llama-shaped summary fields: the widest layer (buffer sizing and the C-ABI's config struct)
    cfg.n_heads = cfg.n_kv_heads = cfg.head_dim = cfg.intermediate_size = 0;
    for (const LayerSpec& L : cfg.layers) {
        cfg.n_heads = std::max(cfg.n_heads, L.heads); cfg.n_kv_heads = std::max(cfg.n_kv_heads, L.kv_heads);
        cfg.head_dim = std::max(cfg.head_dim, L.dim); cfg.intermediate_size = std::max(cfg.intermediate_size, L.ff);
    }
    cfg.max_seq_len = 4096;
    return true;
}

std::vector<TensorBinding> tensors(const ModelConfig& cfg) {
    std::vector<TensorBinding> t;
    const int W = cfg.hidden_size;
    t.push_back({"embed", TensorSlot::EMBED, -1, cfg.vocab_size, W});
    t.push_back({"final.norm", TensorSlot::OUT_NORM, -1, 1, W});
    t.push_back({"head", TensorSlot::HEAD, -1, cfg.vocab_size, W});
    for (int i = 0; i < cfg.n_layers; i++) {
        const LayerSpec& L = cfg.layers[(size_t)i];
        if (L.weights_of >= 0) continue;
        const std::string p = "l" + std::to_string(i) + ".";
        const int qd = L.heads * L.dim, kd = L.kv_heads * L.dim, vd = L.kv_heads * L.vdim, od = L.heads * L.vdim;
        t.push_back({p + "norm1", TensorSlot::NORM1, i, 1, W});
        t.push_back({p + "mix.q", TensorSlot::WQ, i, qd, W});
        t.push_back({p + "mix.k", TensorSlot::WK, i, kd, W});
        t.push_back({p + "mix.v", TensorSlot::WV, i, vd, W});
        t.push_back({p + "mix.q.norm", TensorSlot::Q_NORM, i, 1, qd});
        t.push_back({p + "mix.k.norm", TensorSlot::K_NORM, i, 1, kd});
        t.push_back({p + "mix.o", TensorSlot::WO, i, W, od});
        t.push_back({p + "ls1", TensorSlot::LS1, i, 1, W});
        if (L.ff > 0) {
            t.push_back({p + "mlp.gate", TensorSlot::GATE, i, L.ff, W});
            t.push_back({p + "mlp.up", TensorSlot::UP, i, L.ff, W});
            t.push_back({p + "mlp.down", TensorSlot::DOWN, i, W, L.ff});
            t.push_back({p + "ls2", TensorSlot::LS2, i, 1, W});
        }
    }
    return t;
}

const ModelFamily kFamily = {"Zelunex", config_from_json, tensors};

}  // namespace

const ModelFamily* zelunex_family() { return &kFamily; }

}}  // namespace nt::b200
