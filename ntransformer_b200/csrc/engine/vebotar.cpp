// vebotar.cpp — the Vebotar family: a decoder over several residual streams (BlockForm::STREAMS) whose mixer is differential
// attention (two softmax maps per head over one set of values, combined as A1 v - lambda * A2 v and re-normalised per head)
// with partial interleaved rotary positions under a long-context frequency blend, a block-local causal mask (LayerSpec::chunk),
// optional reuse of an earlier layer's key / value cache (LayerSpec::kv_from), and whose feed-forward is a routed mixture of
// squared-ReLU experts plus a sigmoid-gated shared expert (FfKind::MOE_RELU2).  The embedding row is scaled by a constant.
// Everything that varies between models of the family is read from config.json; absent optional objects (rot, rot.scaling,
// mask, mlp, mlp.shared, streams, embedding) switch their mechanism off.
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
    cfg.streams = 0;
    if (root.has("streams") && !root.at("streams").is_null()) {
        if (!need_int(root, "streams", cfg.streams, err, "config") || cfg.streams < 1 || cfg.streams > 16) { if (err.empty()) err = "config: \"streams\" must be 1..16"; return false; }
    }
    cfg.embed_scale = 1.0f;
    if (root.has("embedding") && root.at("embedding").is_object() && root.at("embedding").has("scale") &&
        !need_float(root.at("embedding"), "scale", cfg.embed_scale, err, "config.embedding")) return false;
    const Json& layers = root.at("layers");
    if (!layers.is_array() || layers.arr.empty()) { err = "config: \"layers\" must be a non-empty list"; return false; }
    cfg.n_layers = (int)layers.arr.size();
    cfg.model_name = "vebotar";
    cfg.bos_token_id = -1; cfg.eos_token_id = -1;
    for (size_t i = 0; i < layers.arr.size(); i++) {
        const Json& e = layers.arr[i];
        const std::string where = "config.layers[" + std::to_string(i) + "]";
        LayerSpec L;
        const std::string type = e.at("type").string_or("");
        if (type != "attention") { err = where + ": mixer type \"" + type + "\" is not part of this family"; return false; }
        L.mixer = MixerKind::ATTN_WINDOW;
        L.form = BlockForm::STREAMS;
        L.qk_norm = QKNorm::NONE;
        L.maps = 2;
        const Json& m = e.at("mixer");
        if (!m.is_object()) { err = where + ": \"mixer\" is missing"; return false; }
        if (!need_int(m, "heads", L.heads, err, where) || !need_int(m, "kv_heads", L.kv_heads, err, where) || !need_int(m, "dim", L.dim, err, where) ||
            !need_int(m, "vdim", L.vdim, err, where) || !need_float(m, "scale", L.scale, err, where) || !need_float(m, "diff", L.diff, err, where))
            return false;
        if (L.heads <= 0 || L.kv_heads <= 0 || L.heads % L.kv_heads || L.dim <= 0 || L.vdim <= 0) { err = where + ": invalid mixer sizes"; return false; }
        if (m.has("mask") && m.at("mask").is_object()) {
            if (!need_int(m.at("mask"), "size", L.chunk, err, where + ".mask") || L.chunk <= 0) { if (err.empty()) err = where + ": invalid mask size"; return false; }
        }
        if (m.has("rot") && m.at("rot").is_object()) {
            const Json& r = m.at("rot");
            if (!need_int(r, "dims", L.rot.dims, err, where + ".rot") || !need_float(r, "base", L.rot.base, err, where + ".rot")) return false;
            if (L.rot.dims < 0 || L.rot.dims > L.dim || (L.rot.dims & 1) || L.rot.base <= 0.f) { err = where + ": rot.dims must be even and at most dim"; return false; }
            L.rot.interleaved = true;
            if (r.has("scaling") && r.at("scaling").is_object()) {
                const Json& sc = r.at("scaling");
                const std::string w2 = where + ".rot.scaling";
                if (!need_float(sc, "factor", L.rot.factor, err, w2) || !need_float(sc, "original", L.rot.original, err, w2) ||
                    !need_float(sc, "fast", L.rot.fast, err, w2) || !need_float(sc, "slow", L.rot.slow, err, w2)) return false;
                if (L.rot.factor <= 0.f || L.rot.original <= 0.f || L.rot.fast <= 0.f || L.rot.slow <= 0.f) { err = w2 + ": values must be positive"; return false; }
            }
        }
        if (m.has("kv_from") && !m.at("kv_from").is_null()) {
            L.kv_from = (int)m.at("kv_from").int_or(-1);
            if (L.kv_from < 0 || L.kv_from >= (int)i || cfg.layers[(size_t)L.kv_from].kv_from >= 0) { err = where + ": \"kv_from\" must name an earlier layer that has key / value projections"; return false; }
            const LayerSpec& J = cfg.layers[(size_t)L.kv_from];
            if (J.kv_heads != L.kv_heads || J.dim != L.dim || J.vdim != L.vdim || J.maps != L.maps) { err = where + ": \"kv_from\" layer has other key / value sizes"; return false; }
        }
        const Json& mlp = e.at("mlp");
        if (mlp.is_null()) L.ff = 0;
        else {
            const std::string kind = mlp.at("kind").string_or("");
            if (kind != "moe") { err = where + ": feed-forward kind \"" + kind + "\" is not part of this family"; return false; }
            L.ff_kind = FfKind::MOE_RELU2;
            if (!need_int(mlp.at("expert"), "ff", L.ff, err, where + ".mlp.expert") || !need_int(mlp.at("router"), "experts", L.experts, err, where + ".mlp.router") ||
                !need_int(mlp.at("router"), "top", L.top, err, where + ".mlp.router")) return false;
            if (L.ff <= 0 || L.experts <= 0 || L.top <= 0 || L.top > L.experts || L.experts > 256) { err = where + ": invalid expert sizes (1 <= top <= experts <= 256)"; return false; }
            if (mlp.has("shared") && mlp.at("shared").is_object()) {
                if (!need_int(mlp.at("shared"), "ff", L.shared_ff, err, where + ".mlp.shared") || L.shared_ff <= 0) { if (err.empty()) err = where + ": invalid shared ff"; return false; }
            }
        }
        cfg.layers.push_back(L);
    }
    cfg.n_heads = cfg.n_kv_heads = cfg.head_dim = cfg.intermediate_size = 0;
    for (const LayerSpec& L : cfg.layers) {
        cfg.n_heads = std::max(cfg.n_heads, L.heads); cfg.n_kv_heads = std::max(cfg.n_kv_heads, L.kv_heads);
        cfg.head_dim = std::max(cfg.head_dim, L.dim); cfg.intermediate_size = std::max(cfg.intermediate_size, std::max(L.ff, L.shared_ff));
    }
    cfg.max_seq_len = 4096;
    return true;
}

std::vector<TensorBinding> tensors(const ModelConfig& cfg) {
    std::vector<TensorBinding> t;
    const int W = cfg.hidden_size, S = cfg.streams;
    t.push_back({"embed", TensorSlot::EMBED, -1, cfg.vocab_size, W});
    t.push_back({"final.norm", TensorSlot::OUT_NORM, -1, 1, W});
    t.push_back({"head", TensorSlot::HEAD, -1, cfg.vocab_size, W});
    for (int i = 0; i < cfg.n_layers; i++) {
        const LayerSpec& L = cfg.layers[(size_t)i];
        const std::string p = "l" + std::to_string(i) + ".";
        const int qd = L.heads * L.maps * L.dim, kd = L.kv_heads * L.maps * L.dim, vd = L.kv_heads * L.vdim, od = L.heads * L.vdim;
        t.push_back({p + "norm1", TensorSlot::NORM1, i, 1, W});
        t.push_back({p + "mix.q", TensorSlot::WQ, i, qd, W});
        if (L.kv_from < 0) {
            t.push_back({p + "mix.k", TensorSlot::WK, i, kd, W});
            t.push_back({p + "mix.v", TensorSlot::WV, i, vd, W});
        }
        t.push_back({p + "mix.lq1", TensorSlot::LQ1, i, 1, L.dim});
        t.push_back({p + "mix.lk1", TensorSlot::LK1, i, 1, L.dim});
        t.push_back({p + "mix.lq2", TensorSlot::LQ2, i, 1, L.dim});
        t.push_back({p + "mix.lk2", TensorSlot::LK2, i, 1, L.dim});
        t.push_back({p + "mix.o", TensorSlot::WO, i, W, od});
        if (S > 0) {
            t.push_back({p + "hc1.in", TensorSlot::HC1_IN, i, 1, S});
            t.push_back({p + "hc1.out", TensorSlot::HC1_OUT, i, 1, S});
            t.push_back({p + "hc1.mix", TensorSlot::HC1_MIX, i, S, S});
        }
        if (L.ff > 0) {
            t.push_back({p + "norm2", TensorSlot::NORM2, i, 1, W});
            t.push_back({p + "mlp.router", TensorSlot::ROUTER, i, L.experts, W});
            for (int e = 0; e < L.experts; e++) {
                const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                t.push_back({q + "up", TensorSlot::EXPERT_UP, i, L.ff, W, e});
                t.push_back({q + "down", TensorSlot::EXPERT_DOWN, i, W, L.ff, e});
            }
            if (L.shared_ff > 0) {
                t.push_back({p + "mlp.shared.up", TensorSlot::SHARED_UP, i, L.shared_ff, W});
                t.push_back({p + "mlp.shared.down", TensorSlot::SHARED_DOWN, i, W, L.shared_ff});
                t.push_back({p + "mlp.shared.sg", TensorSlot::SHARED_GATE, i, 1, W});
            }
            if (S > 0) {
                t.push_back({p + "hc2.in", TensorSlot::HC2_IN, i, 1, S});
                t.push_back({p + "hc2.out", TensorSlot::HC2_OUT, i, 1, S});
                t.push_back({p + "hc2.mix", TensorSlot::HC2_MIX, i, S, S});
            }
        }
    }
    return t;
}

const ModelFamily kFamily = {"Vebotar", config_from_json, tensors};

}  // namespace

const ModelFamily* vebotar_family() { return &kFamily; }

}}  // namespace nt::b200
