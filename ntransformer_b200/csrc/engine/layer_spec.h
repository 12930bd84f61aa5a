// layer_spec.h — what one decoder layer is made of, for model families described layer by layer (a folder with config.json +
// model.safetensors) instead of by the fixed Llama block of the GGUF families.  Every mechanism is a parameter here so that
// another family can combine them differently; a Llama block would read {ROPE_CAUSAL mixer, sequential block, SiLU GLU}.
#pragma once
#include <string>
#include <vector>

namespace nt { namespace b200 {

enum class MixerKind { ATTN_ROPE_CAUSAL = 0,     // rotary positions, full causal mask (the GGUF Llama block)
                       ATTN_WINDOW = 1 };        // no positions in the scores; sliding window + kept first tokens; soft-capped scores
enum class QKNorm { NONE = 0, WHOLE = 1 };       // WHOLE: one RMS norm across ALL heads of the projection (gain vector of that length)
enum class GluAct { SILU = 0, GELU_TANH = 1 };
enum class BlockForm { SEQUENTIAL = 0,           // x += mixer(norm1 x) ; x += ff(norm2 x)
                       PARALLEL = 1 };           // h = norm1 x ; x += m * (ls1 * mixer(h) + ls2 * ff(h))

struct LayerSpec {
    MixerKind mixer = MixerKind::ATTN_ROPE_CAUSAL;
    BlockForm form = BlockForm::SEQUENTIAL;
    int heads = 0, kv_heads = 0;
    int dim = 0;                 // per-head query/key width
    int vdim = 0;                // per-head value width
    float scale = 0.f;           // score multiplier
    float softcap = 0.f;         // score <- softcap * tanh(score / softcap); 0 = none
    int window = 0;              // key j visible from i iff j <= i and (i - j < window or j < keep_first); 0 = full causal
    int keep_first = 0;
    QKNorm qk_norm = QKNorm::NONE;
    int ff = 0;                  // feed-forward width; 0 = the layer has no feed-forward
    GluAct act = GluAct::SILU;
    bool layer_scale = false;    // per-channel gains on each branch before the residual sum
    int weights_of = -1;         // >= 0: this layer reads that layer's tensors (own KV cache)
};

}}  // namespace nt::b200
