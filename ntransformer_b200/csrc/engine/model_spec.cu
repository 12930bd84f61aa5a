// model_spec.cu — the resident model for families described layer by layer (engine/layer_spec.h, engine/model_registry.h):
// loading a model folder, the per-token decode step and the batched prompt pass, written against LayerSpec so that the
// mechanisms (windowed / soft-capped attention, whole-projection q/k norm, parallel block with layer scale, GELU-gated unit,
// layers sharing tensors) combine freely.  Same buffers, stream, CUDA-graph replay, logits and sampler as the GGUF families
// (engine/model.cu); the KV cache is per layer because layers may differ in width.
//
// Arithmetic: the residual stream, norms, softmax and every accumulation are F32.  Weights stay in their stored dtype (BF16)
// and are widened in registers, or — exact 32-bit mode — are widened once at load.  The cache stores BF16 (F32 in exact mode).
//
// Launches per layer and decoded token (6):  [RMS norm + q/k/v GEMV, one launch]  [q/k norm + cache write]  [window attention]
//   [RMS norm + gate/up GEMV + GELU gate]  [o GEMV: x += m * ls1 * .]  [down GEMV: x += m * ls2 * .]   — the block norm lives in
//   the GEMV prologues, every residual update, gain and activation in a GEMV epilogue.
#include "model.h"
#include "safetensors.h"

#include <algorithm>
#include <chrono>
#include <cstring>
#include <sys/stat.h>

namespace nt { namespace b200 {

namespace {
template <typename T> T* dmalloc(size_t n) {
    T* p = nullptr;
    NT_CUDA_CHECK(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
    return p;
}
__global__ void iota_spec_kernel(int* out, int first, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = first + i;
}
constexpr int SPEC_PREFILL_CHUNK = 2048;
GemvMat mat_of(const Weight& w, float* y) { GemvMat m; m.W = w.ptr; m.y = y; m.out = w.rows; m.dtype = w.dtype; m.row_pitch = w.pitch; return m; }
}  // namespace

bool Model::load(const std::string& path, int max_context) {
    struct stat st;
    if (stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) return load_dir(path, max_context);
    return load_gguf(path, max_context);
}

bool Model::bind_slot(TensorSlot slot, int layer, const void* ptr, DType dt, int rows, int cols, size_t pitch) {
    auto W = [&](Weight& w) {
        if (!dense_dtype(dt)) return false;
        w.ptr = ptr; w.dtype = dt; w.rows = rows; w.cols = cols; w.pitch = pitch ? pitch : dtype_row_size(dt, (size_t)cols); w.owned = false;
        return true;
    };
    auto V = [&](const float*& v) { if (dt != DType::F32) return false; v = static_cast<const float*>(ptr); return true; };
    if (slot == TensorSlot::EMBED) return W(embd_);
    if (slot == TensorSlot::HEAD) return W(head_);
    if (slot == TensorSlot::OUT_NORM) return V(out_norm_);
    if (layer < 0 || layer >= cfg_.n_layers) return false;
    LayerWeights& L = layers_[(size_t)layer];
    switch (slot) {
        case TensorSlot::NORM1: return V(L.attn_norm);
        case TensorSlot::NORM2: return V(L.ffn_norm);
        case TensorSlot::Q_NORM: return V(L.q_norm);
        case TensorSlot::K_NORM: return V(L.k_norm);
        case TensorSlot::LS1: return V(L.ls1);
        case TensorSlot::LS2: return V(L.ls2);
        case TensorSlot::WQ: return W(L.wq);
        case TensorSlot::WK: return W(L.wk);
        case TensorSlot::WV: return W(L.wv);
        case TensorSlot::WO: return W(L.wo);
        case TensorSlot::GATE: return W(L.gate);
        case TensorSlot::UP: return W(L.up);
        case TensorSlot::DOWN: return W(L.down);
        default: return false;
    }
}

// config.json -> family -> LayerSpecs; model.safetensors -> one device arena.  Matrices keep their stored dtype (widened to F32
// in exact mode), gain vectors always become F32.  Shapes are checked against the configuration before anything is uploaded.
bool Model::load_dir(const std::string& dir, int max_context) {
    const auto t_start = std::chrono::steady_clock::now();
    fprintf(stderr, "Loading model folder: %s\n", dir.c_str());
    ModelConfig cfg;
    const ModelFamily* fam = nullptr;
    if (!read_model_dir(dir, cfg, &fam)) return false;
    cfg.max_seq_len = std::max(1, max_context);
    cfg.print();
    SafeTensorsFile f;
    if (!f.open(dir + "/model.safetensors")) return false;
    init(cfg, 0, 1);
    const std::vector<TensorBinding> plan = fam->tensors(cfg_);
    struct Job { const SafeTensorInfo* ti; const TensorBinding* b; size_t off; DType dst; };
    std::vector<Job> jobs;
    size_t arena = 0, stage_max = 0;
    for (const TensorBinding& b : plan) {
        const SafeTensorInfo* ti = f.find(b.name);
        if (!ti) { fprintf(stderr, "model: tensor not found: %s\n", b.name.c_str()); return false; }
        const bool vec = b.rows == 1 && ti->shape.size() == 1;
        if (!dense_dtype(ti->dtype) || !(vec ? ti->shape[0] == b.cols : (ti->shape.size() == 2 && ti->shape[0] == b.rows && ti->shape[1] == b.cols))) {
            fprintf(stderr, "model: tensor %s does not have the shape the configuration needs [%d x %d]\n", b.name.c_str(), b.rows, b.cols);
            return false;
        }
        const bool is_vec = b.slot == TensorSlot::OUT_NORM || b.slot == TensorSlot::NORM1 || b.slot == TensorSlot::NORM2 || b.slot == TensorSlot::Q_NORM ||
                            b.slot == TensorSlot::K_NORM || b.slot == TensorSlot::LS1 || b.slot == TensorSlot::LS2;
        const DType dst = (is_vec || exact32_) ? DType::F32 : ti->dtype;
        jobs.push_back({ti, &b, arena, dst});
        arena += ((size_t)b.rows * b.cols * dtype_size(dst) + 255) & ~(size_t)255;
        stage_max = std::max(stage_max, (size_t)(ti->end - ti->begin));
    }
    uint8_t* base = nullptr;
    if (cudaMalloc(&base, std::max<size_t>(arena, 256)) != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "model: cannot allocate %.2f GB of device memory for the weights\n", arena / 1e9);
        return false;
    }
    owned_.push_back(base);
    cudaStream_t st = nullptr;
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    uint8_t* host = nullptr;
    NT_CUDA_CHECK(cudaHostAlloc((void**)&host, std::max<size_t>(stage_max, 16), cudaHostAllocDefault));
    uint8_t* dev_stage = dmalloc<uint8_t>(stage_max);
    bool ok = true;
    for (const Job& j : jobs) {
        const size_t bytes = (size_t)(j.ti->end - j.ti->begin), n = (size_t)j.b->rows * j.b->cols;
        if (!f.read(*j.ti, host)) { fprintf(stderr, "model: short read of %s\n", j.b->name.c_str()); ok = false; break; }
        if (j.dst == j.ti->dtype) NT_CUDA_CHECK(cudaMemcpyAsync(base + j.off, host, bytes, cudaMemcpyHostToDevice, st));
        else {
            NT_CUDA_CHECK(cudaMemcpyAsync(dev_stage, host, bytes, cudaMemcpyHostToDevice, st));
            dense_to_f32(reinterpret_cast<float*>(base + j.off), dev_stage, j.ti->dtype, n, st);
        }
        NT_CUDA_CHECK(cudaStreamSynchronize(st));          // the staging buffers are reused by the next tensor
        if (!bind_slot(j.b->slot, j.b->layer, base + j.off, j.dst, j.b->rows, j.b->cols, 0)) { fprintf(stderr, "model: cannot bind %s\n", j.b->name.c_str()); ok = false; break; }
    }
    cudaFreeHost(host);
    cudaFree(dev_stage);
    cudaStreamDestroy(st);
    if (!ok || !finalize()) return false;
    load_seconds_ = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
    fprintf(stderr, "  Loaded %d layers (%s weights, %s cache): %.3f GB resident, %.2f s\nModel loaded successfully!\n", cfg_.n_layers,
            exact32_ ? "F32" : "stored-dtype", dtype_name(cache_dt_), arena / 1e9, load_seconds_);
    return true;
}

bool Model::finalize_spec() {
    const int hidden = cfg_.hidden_size, max_seq = cfg_.max_seq_len;
    if (!embd_.ptr || !out_norm_ || !head_.ptr) { fprintf(stderr, "model: embedding / final norm / head missing\n"); return false; }
    int qmax = 1, kmax = 1, vmax = 1, omax = 1, ffmax = 1;
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerSpec& S = cfg_.layers[(size_t)i];
        const LayerWeights& L = layer_weights(i);
        const bool mlp_ok = S.ff == 0 || (L.gate.ptr && L.up.ptr && L.down.ptr && (!S.layer_scale || L.ls2));
        if (!L.attn_norm || !L.wq.ptr || !L.wk.ptr || !L.wv.ptr || !L.wo.ptr || !mlp_ok || (S.layer_scale && !L.ls1) ||
            (S.qk_norm == QKNorm::WHOLE && (!L.q_norm || !L.k_norm))) {
            fprintf(stderr, "model: layer %d is missing tensors\n", i);
            return false;
        }
        if (S.mixer != MixerKind::ATTN_WINDOW || S.form != BlockForm::PARALLEL) { fprintf(stderr, "model: layer %d: this mixer / block form has no layer-spec kernels yet\n", i); return false; }
        if (S.vdim > 256) { fprintf(stderr, "model: layer %d: value heads wider than 256 are not covered\n", i); return false; }
        qmax = std::max(qmax, S.heads * S.dim); kmax = std::max(kmax, S.kv_heads * S.dim); vmax = std::max(vmax, S.kv_heads * S.vdim);
        omax = std::max(omax, S.heads * S.vdim); ffmax = std::max(ffmax, S.ff);
    }
    cache_dt_ = exact32_ ? DType::F32 : DType::BF16;
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    hidden_ = dmalloc<float>(hidden);
    xnorm_ = dmalloc<float>(hidden);
    q_ = dmalloc<float>(qmax); k_ = dmalloc<float>(kmax); v_ = dmalloc<float>(vmax); attn_ = dmalloc<float>(omax);
    act_ = dmalloc<float>(ffmax);
    logits_ = dmalloc<float>(cfg_.vocab_size);
    NT_CUDA_CHECK(cudaMemset(logits_, 0, sizeof(float) * (size_t)cfg_.vocab_size));
    kcs_.assign((size_t)cfg_.n_layers, nullptr);
    vcs_.assign((size_t)cfg_.n_layers, nullptr);
    const size_t es = dtype_size(cache_dt_);
    for (int i = 0; i < cfg_.n_layers; i++) {          // every layer RUN owns a cache, also one that borrows its tensors
        const LayerSpec& S = cfg_.layers[(size_t)i];
        const size_t kb = es * max_seq * S.kv_heads * S.dim, vb = es * max_seq * S.kv_heads * S.vdim;
        if (cudaMalloc(&kcs_[(size_t)i], std::max<size_t>(kb, 16)) != cudaSuccess || cudaMalloc(&vcs_[(size_t)i], std::max<size_t>(vb, 16)) != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "model: cannot allocate the KV cache for %d tokens\n", max_seq);
            return false;
        }
        NT_CUDA_CHECK(cudaMemset(kcs_[(size_t)i], 0, std::max<size_t>(kb, 16)));
        NT_CUDA_CHECK(cudaMemset(vcs_[(size_t)i], 0, std::max<size_t>(vb, 16)));
    }
    step_dev_ = dmalloc<int>(2);
    argmax_dev_ = dmalloc<int>(1);
    NT_CUDA_CHECK(cudaMallocHost(&argmax_host_, sizeof(int)));
    prefill_min_tokens_ = 16;
    finalized_ = true;
    return true;
}

static WindowAttn attn_of(const LayerSpec& S) {
    WindowAttn a;
    a.heads = S.heads; a.kv_heads = S.kv_heads; a.dim = S.dim; a.vdim = S.vdim; a.window = S.window; a.keep = S.keep_first; a.scale = S.scale; a.softcap = S.softcap;
    return a;
}

void Model::step_body_spec(cudaStream_t s) {
    const int hidden = cfg_.hidden_size;
    const int* pos_dev = step_dev_ + 1;
    const float m = cfg_.residual_mult;
    embed_rows(hidden_, embd_.ptr, embd_.dtype, step_dev_, 1, hidden, s);
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerSpec& S = cfg_.layers[(size_t)i];
        const LayerWeights& L = layer_weights(i);
        // Both branches read norm(x) of the x the layer started from.  The q/k/v and the gate/up launches each normalise hidden_ in
        // their prologue (bit-identical results), and both run before the first epilogue that updates hidden_.
        GemvMat qkv[3] = {mat_of(L.wq, q_), mat_of(L.wk, k_), mat_of(L.wv, v_)};
        gemv_dense(qkv, 3, hidden, hidden_, DENSE_STORE, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps);
        qk_norm_kv_write(q_, k_, v_, L.q_norm, L.k_norm, cfg_.norm_eps, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, 1, pos_dev, 0, S.heads * S.dim,
                         S.kv_heads * S.dim, S.kv_heads * S.vdim, s);
        attention_window(attn_, q_, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, 1, pos_dev, 0, cfg_.max_seq_len, attn_of(S), s);
        if (S.ff > 0) {
            GemvMat gu[2] = {mat_of(L.gate, act_), mat_of(L.up, nullptr)};
            gemv_dense(gu, 2, hidden, hidden_, S.act == GluAct::GELU_TANH ? DENSE_GEGLU : DENSE_SWIGLU, nullptr, 1.f, s, L.attn_norm, cfg_.norm_eps);
        }
        GemvMat o = mat_of(L.wo, hidden_);
        gemv_dense(&o, 1, S.heads * S.vdim, attn_, DENSE_SCALED_ADD, L.ls1, m, s);
        if (S.ff > 0) {
            GemvMat d = mat_of(L.down, hidden_);
            gemv_dense(&d, 1, S.ff, act_, DENSE_SCALED_ADD, L.ls2, m, s);
        }
    }
}

void Model::step_head_spec(cudaStream_t s) {
    GemvMat h = mat_of(head_, logits_);
    gemv_dense(&h, 1, cfg_.hidden_size, hidden_, DENSE_STORE, nullptr, 1.f, s, out_norm_, cfg_.norm_eps);       // final norm in the prologue
}

void Model::ensure_prefill_buffers_spec(int tokens) {
    if (tokens <= pf_.cap) return;
    NT_CUDA_CHECK(cudaStreamSynchronize(stream_));
    for (void* p : {(void*)pf_.x, (void*)pf_.q, (void*)pf_.k, (void*)pf_.v, (void*)pf_.attn, (void*)pf_.g, (void*)pf_.u, (void*)pf_.h, (void*)pf_.tmp,
                    pf_.ws, pf_.ws2, pf_.hws, (void*)pf_.tok})
        if (p) cudaFree(p);
    const size_t T = (size_t)((tokens + 127) / 128 * 128), hidden = (size_t)cfg_.hidden_size;
    size_t qmax = 1, kmax = 1, vmax = 1, omax = 1, ffmax = 1;
    for (const LayerSpec& S : cfg_.layers) {
        qmax = std::max(qmax, (size_t)S.heads * S.dim); kmax = std::max(kmax, (size_t)S.kv_heads * S.dim); vmax = std::max(vmax, (size_t)S.kv_heads * S.vdim);
        omax = std::max(omax, (size_t)S.heads * S.vdim); ffmax = std::max(ffmax, (size_t)S.ff);
    }
    pf_.x = dmalloc<float>(T * hidden); pf_.h = dmalloc<float>(T * hidden); pf_.tmp = dmalloc<float>(T * hidden);
    pf_.q = dmalloc<float>(T * qmax); pf_.k = dmalloc<float>(T * kmax); pf_.v = dmalloc<float>(T * vmax); pf_.attn = dmalloc<float>(T * omax);
    pf_.g = dmalloc<float>(T * ffmax); pf_.u = dmalloc<float>(T * ffmax);
    pf_.tok = dmalloc<int>(T);
    pf_.ws = pf_.ws2 = pf_.hws = nullptr;
    bool any_tc = false;
    for (int i = 0; i < cfg_.n_layers; i++) {
        const LayerWeights& L = layer_weights(i);
        for (const Weight* w : {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down}) any_tc = any_tc || (w->ptr && spec_tc_ok(*w));
    }
    if (any_tc) {                         // BF16 hi/lo splits of the three GEMM inputs (normed block input, attention output, gated activation)
        pf_.hws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)hidden));
        pf_.ws = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)omax));
        pf_.ws2 = dmalloc<uint8_t>(gemm_f16_tc_workspace_bytes((int)T, (int)ffmax));
    }
    pf_.cap = (int)T;
}

// BF16 rows that the tcgen05 GEMM can read in place through TMA (rows % 128, cols % 64, 16-byte aligned); never in exact mode.
bool Model::spec_tc_ok(const Weight& w) const {
    static const bool off = getenv("NT_B200_NO_TC_PREFILL") != nullptr;
    return !exact32_ && !off && w.dtype == DType::BF16 && gemm_f16_tc_supported(w.ptr, w.rows, w.cols, w.pitch);
}

// C (ep)= A . W^T for T prompt rows: on the tensor cores from the BF16 hi/lo split of A when the matrix qualifies, else in FP32
// on CUDA cores from A itself.  Either input may be null when the caller knows which path the matrix takes.
void Model::spec_gemm(float* C, const float* A, const void* A_split, const Weight& w, int T, DenseEpilogue ep, const float* row_scale, float alpha, cudaStream_t s) {
    if (A_split && spec_tc_ok(w)) {
        TcOpts o;
        o.bf16 = true;
        if (ep == DENSE_SCALED_ADD) { o.col_scale = row_scale; o.alpha = alpha; }
        NT_CHECK(gemm_f16_tc_ws(C, A_split, w.ptr, T, w.rows, w.cols, ep != DENSE_STORE, s, o), "prefill GEMM rejected");
        return;
    }
    NT_CHECK(A != nullptr, "spec_gemm: the FP32 input of a CUDA-core GEMM is missing");
    gemm_dense(C, A, w.ptr, w.dtype, w.pitch, T, w.rows, w.cols, ep, row_scale, alpha, s);
}

// A prompt (or a portion of one: start_pos > 0) in chunks of up to SPEC_PREFILL_CHUNK tokens.  The chunk's key / value rows go to
// the cache first, then the attention kernel reads cache rows only — earlier portions, the kept first tokens and the chunk itself
// alike — so where a prompt is cut cannot change what a query sees.
void Model::prefill_spec(const int* tokens, int seq_len, int start_pos) {
    cudaStream_t s = stream_;
    const int hidden = cfg_.hidden_size;
    const float m = cfg_.residual_mult;
    ensure_prefill_buffers_spec(std::min(seq_len, SPEC_PREFILL_CHUNK));
    int last_rows = 0;
    for (int c0 = 0; c0 < seq_len; c0 += SPEC_PREFILL_CHUNK) {
        const int T = std::min(SPEC_PREFILL_CHUNK, seq_len - c0), p0 = start_pos + c0;
        last_rows = T;
        NT_CUDA_CHECK(cudaMemcpyAsync(pf_.tok, tokens + c0, sizeof(int) * (size_t)T, cudaMemcpyHostToDevice, s));
        embed_rows(pf_.x, embd_.ptr, embd_.dtype, pf_.tok, T, hidden, s);
        for (int i = 0; i < cfg_.n_layers; i++) {
            const LayerSpec& S = cfg_.layers[(size_t)i];
            const LayerWeights& L = layer_weights(i);
            // the block's normed input feeds q, k, v, gate and up: as FP32 rows, as a BF16 split, or both, by what those matrices take
            bool h_f32 = false, h_split = false;
            auto reads_h = [&](const Weight& w) { if (spec_tc_ok(w)) h_split = true; else h_f32 = true; };
            reads_h(L.wq); reads_h(L.wk); reads_h(L.wv);
            if (S.ff > 0) { reads_h(L.gate); reads_h(L.up); }
            if (h_f32) rmsnorm(pf_.h, pf_.x, L.attn_norm, T, hidden, cfg_.norm_eps, s);
            if (h_split) rmsnorm_split(pf_.hws, pf_.x, L.attn_norm, T, hidden, cfg_.norm_eps, s, true);
            const float* hf = h_f32 ? pf_.h : nullptr;
            const void* hs = h_split ? pf_.hws : nullptr;
            spec_gemm(pf_.q, hf, hs, L.wq, T, DENSE_STORE, nullptr, 1.f, s);
            spec_gemm(pf_.k, hf, hs, L.wk, T, DENSE_STORE, nullptr, 1.f, s);
            spec_gemm(pf_.v, hf, hs, L.wv, T, DENSE_STORE, nullptr, 1.f, s);
            qk_norm_kv_write(pf_.q, pf_.k, pf_.v, L.q_norm, L.k_norm, cfg_.norm_eps, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, T, nullptr, p0,
                             S.heads * S.dim, S.kv_heads * S.dim, S.kv_heads * S.vdim, s);
            attention_window(pf_.attn, pf_.q, kcs_[(size_t)i], vcs_[(size_t)i], cache_dt_, T, nullptr, p0, cfg_.max_seq_len, attn_of(S), s);
            const bool o_tc = spec_tc_ok(L.wo);
            if (o_tc) split_activations(pf_.ws, pf_.attn, T, S.heads * S.vdim, s, true);
            spec_gemm(pf_.x, pf_.attn, o_tc ? pf_.ws : nullptr, L.wo, T, DENSE_SCALED_ADD, L.ls1, m, s);
            if (S.ff > 0) {
                const bool gelu = S.act == GluAct::GELU_TANH, down_tc = spec_tc_ok(L.down);
                if (spec_tc_ok(L.gate) && spec_tc_ok(L.up) && down_tc) {
                    // gate / up GEMMs with the gated activation and the split for the down projection in the epilogue: the
                    // [T, ff] activations never reach HBM in FP32
                    TcOpts o; o.bf16 = true; o.gelu = gelu;
                    NT_CHECK(gemm_f16_tc_swiglu_ws(pf_.ws2, pf_.hws, L.gate.ptr, L.up.ptr, T, S.ff, hidden, s, o), "prefill GEMM (gate/up) rejected");
                } else {
                    spec_gemm(pf_.g, hf, hs, L.gate, T, DENSE_STORE, nullptr, 1.f, s);
                    spec_gemm(pf_.u, hf, hs, L.up, T, DENSE_STORE, nullptr, 1.f, s);
                    glu_mul(pf_.g, pf_.g, pf_.u, (size_t)T * S.ff, gelu, s);
                    if (down_tc) split_activations(pf_.ws2, pf_.g, T, S.ff, s, true);
                }
                spec_gemm(pf_.x, pf_.g, down_tc ? pf_.ws2 : nullptr, L.down, T, DENSE_SCALED_ADD, L.ls2, m, s);
            }
        }
        if (!want_.empty()) emit_wanted(pf_.x, c0, T, s);
    }
    copy(hidden_, pf_.x + (size_t)(last_rows - 1) * hidden, hidden, s);
    step_head(s);
}

}}  // namespace nt::b200
