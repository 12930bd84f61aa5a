// attention_diff.cu — the pieces around attention_window.cu that differential attention with rotary positions needs:
//   rope_partial_kv_write   rotates the first `dims` channels of every dim-wide head (every map of every head is such a head) of the
//                           query rows in place and of the key rows on their way into the cache; writes the value rows to the cache.
//                           angle = position * freq[i] (F32), cos and sin times `mag`; the frequency table (with its long-context
//                           blend) is made once per layer on the host.
//   diff_combine            o = a1 - lambda * a2 per head from the two maps' outputs, weightless RMS norm over the head, times (1 - diff).
//   streams_*               several residual streams: spread the embedding, read a blend, write back through the mixing matrix.
// The attention itself is attention_window's kernel with WindowAttn::maps = 2 and WindowAttn::chunk.  All F32; compiled WITHOUT
// --use_fast_math (sincosf / expf / division at full precision).
#include "kernels_internal.h"
#include "ring.cuh"
#include <cuda_bf16.h>
#include <algorithm>
#include <cmath>

namespace nt { namespace b200 {

namespace {

__device__ __forceinline__ void cst(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void cst(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// the rotated value of channel c (c < dims) of the head starting at `head`
__device__ __forceinline__ float rotated(const float* head, int c, int dims, bool interleaved, float pos, const float* __restrict__ freq, float mag) {
    const int half = dims >> 1;
    const int i = interleaved ? (c >> 1) : (c < half ? c : c - half);
    const bool first = interleaved ? !(c & 1) : c < half;
    const int c0 = interleaved ? 2 * i : i, c1 = interleaved ? 2 * i + 1 : i + half;
    float sn, cs;
    sincosf(pos * freq[i], &sn, &cs);
    sn *= mag; cs *= mag;
    const float u = head[c0], v = head[c1];
    return first ? u * cs - v * sn : v * cs + u * sn;
}

template <typename KT>
__global__ void __launch_bounds__(256) rope_partial_kv_write_kernel(float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                                                    const float* __restrict__ freq, float mag, int dims, int interleaved, int dim,
                                                                    KT* __restrict__ kc, KT* __restrict__ vc, const int* __restrict__ pos_dev, int p0,
                                                                    int qdim, int kdim, int vdim) {
    extern __shared__ float rq[];            // rotated query channels [qdim / dim][dims]
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int pos = (pos_dev ? *pos_dev : p0) + t;
    const float fp = (float)pos;
    float* q = Q + (size_t)t * qdim;
    const int nq = (qdim / dim) * dims;
    for (int e = threadIdx.x; e < nq; e += 256) { const int h = e / dims, c = e % dims; rq[e] = rotated(q + (size_t)h * dim, c, dims, interleaved, fp, freq, mag); }
    __syncthreads();
    for (int e = threadIdx.x; e < nq; e += 256) { const int h = e / dims, c = e % dims; q[(size_t)h * dim + c] = rq[e]; }
    if (!K) return;
    const float* k = K + (size_t)t * kdim;
    for (int e = threadIdx.x; e < kdim; e += 256) {
        const int h = e / dim, c = e % dim;
        cst(kc, (size_t)pos * kdim + e, c < dims ? rotated(k + (size_t)h * dim, c, dims, interleaved, fp, freq, mag) : k[e]);
    }
    const float* v = V + (size_t)t * vdim;
    for (int e = threadIdx.x; e < vdim; e += 256) cst(vc, (size_t)pos * vdim + e, v[e]);
}

__global__ void __launch_bounds__(256) diff_combine_kernel(float* __restrict__ out, const float* __restrict__ A, const float* __restrict__ lq1,
                                                           const float* __restrict__ lk1, const float* __restrict__ lq2, const float* __restrict__ lk2,
                                                           int n_l, float diff, float eps, int heads, int vdim) {
    __shared__ float red[8];
    __shared__ float lam_s, inv_s;
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    if (warp == 0) {
        float d1 = 0.f, d2 = 0.f;
        for (int i = lane; i < n_l; i += 32) { d1 = fmaf(lq1[i], lk1[i], d1); d2 = fmaf(lq2[i], lk2[i], d2); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { d1 += __shfl_xor_sync(0xFFFFFFFFu, d1, o); d2 += __shfl_xor_sync(0xFFFFFFFFu, d2, o); }
        if (lane == 0) lam_s = expf(d1) - expf(d2) + diff;
    }
    __syncthreads();
    const float lam = lam_s;
    const float* a1 = A + ((size_t)t * heads + h) * 2 * vdim;
    const float* a2 = a1 + vdim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < vdim; i += 256) { const float o = a1[i] - lam * a2[i]; ss = fmaf(o, o, ss); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < 8; w++) tot += red[w];
        inv_s = (1.0f - diff) / sqrtf(tot / (float)vdim + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    float* o = out + ((size_t)t * heads + h) * vdim;
    for (int i = threadIdx.x; i < vdim; i += 256) o[i] = (a1[i] - lam * a2[i]) * inv;
}

constexpr int MAX_STREAMS = 16;

__global__ void streams_spread_kernel(float* __restrict__ X, const float* __restrict__ e, float scale, size_t n, int S, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / width, c = i % width;
    const float v = e[i] * scale;
    for (int s = 0; s < S; s++) X[(t * S + s) * width + c] = v;
}
__global__ void streams_read_kernel(float* __restrict__ u, const float* __restrict__ X, const float* __restrict__ a, size_t n, int S, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / width, c = i % width;
    float acc = 0.f;
    for (int s = 0; s < S; s++) { const float x = X[(t * S + s) * width + c]; acc = a ? fmaf(a[s], x, acc) : acc + x; }
    u[i] = acc;
}
// NS > 0: the number of streams is a compile-time constant (registers, S*S multiply-adds); NS == 0: any S <= MAX_STREAMS
template <int NS>
__global__ void streams_write_kernel(float* __restrict__ X, const float* __restrict__ y, const float* __restrict__ M, const float* __restrict__ b,
                                     size_t n, int S_rt, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / width, c = i % width;
    const float yv = y[i];
    if (NS > 0) {
        float x[NS > 0 ? NS : 1];
#pragma unroll
        for (int s = 0; s < NS; s++) x[s] = X[(t * NS + s) * width + c];
#pragma unroll
        for (int to = 0; to < NS; to++) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < NS; s++) acc = fmaf(M[s * NS + to], x[s], acc);
            X[(t * NS + to) * width + c] = fmaf(b[to], yv, acc);
        }
        return;
    }
    const int S = S_rt;
    float x[MAX_STREAMS], r[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; s++) x[s] = s < S ? X[(t * S + s) * width + c] : 0.f;
#pragma unroll
    for (int to = 0; to < MAX_STREAMS; to++) {
        float acc = 0.f;
        if (to < S) {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; s++) if (s < S) acc = fmaf(M[s * S + to], x[s], acc);
            acc = fmaf(b[to], yv, acc);
        }
        r[to] = acc;
    }
#pragma unroll
    for (int to = 0; to < MAX_STREAMS; to++) if (to < S) X[(t * S + to) * width + c] = r[to];
}
__global__ void scale_rows_kernel(float* __restrict__ x, float scale, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= scale;
}

}  // namespace

float rotary_table(float* freq, int dims, float base, float factor, float original, float fast, float slow) {
    const int half = dims / 2;
    const double lnb = std::log((double)base), two_pi = 6.283185307179586476925;
    // the (fractional) pair index whose wavelength fits `t` times into `original` positions
    auto turn = [&](double t) { return dims * std::log((double)original / (two_pi * t)) / (2.0 * lnb); };
    double lo = 0.0, hi = 0.0;
    if (factor > 0.f) { lo = std::max(std::floor(turn(fast)), 0.0); hi = std::min(std::ceil(turn(slow)), (double)(dims - 1)); }
    for (int i = 0; i < half; i++) {
        double f = std::exp(-2.0 * i / dims * lnb);
        if (factor > 0.f) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            f = f / factor * ramp + f * (1.0 - ramp);
        }
        freq[i] = (float)f;
    }
    return factor > 0.f ? (float)(0.1 * std::log((double)factor) + 1.0) : 1.f;
}

void rope_partial_kv_write(float* Q, const float* K, const float* V, const float* freq, float mag, int dims, bool interleaved, int dim,
                           void* kc, void* vc, DType cache_dt, int tokens, const int* pos_dev, int p0, int qdim, int kdim, int vdim, cudaStream_t s) {
    NT_CHECK(cache_dt == DType::F32 || cache_dt == DType::BF16, "rope_partial_kv_write: F32 or BF16 cache");
    NT_CHECK(dims >= 0 && dims <= dim && !(dims & 1) && qdim % dim == 0 && (!K || kdim % dim == 0), "rope_partial_kv_write: bad sizes");
    if (tokens <= 0) return;
    const size_t smem = sizeof(float) * (size_t)std::max(1, (qdim / dim) * dims);
    NT_CHECK(smem <= 48 * 1024, "rope_partial_kv_write: rotated query channels exceed shared memory");
    if (cache_dt == DType::F32)
        launch_k(rope_partial_kv_write_kernel<float>, dim3(tokens), dim3(256), smem, s, Q, K, V, freq, mag, dims, interleaved ? 1 : 0, dim,
                 static_cast<float*>(kc), static_cast<float*>(vc), pos_dev, p0, qdim, kdim, vdim);
    else
        launch_k(rope_partial_kv_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), smem, s, Q, K, V, freq, mag, dims, interleaved ? 1 : 0, dim,
                 static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), pos_dev, p0, qdim, kdim, vdim);
    count_launch();
}

void diff_combine(float* out, const float* A, const float* lq1, const float* lk1, const float* lq2, const float* lk2, int n_l, float diff,
                  float eps, int tokens, int heads, int vdim, cudaStream_t s) {
    if (tokens <= 0) return;
    launch_k(diff_combine_kernel, dim3(tokens, heads), dim3(256), 0, s, out, A, lq1, lk1, lq2, lk2, n_l, diff, eps, heads, vdim);
    count_launch();
}

void streams_spread(float* X, const float* e, float scale, int tokens, int S, int width, cudaStream_t s) {
    const size_t n = (size_t)tokens * width;
    if (!n) return;
    launch_k(streams_spread_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, X, e, scale, n, S, width);
    count_launch();
}
void streams_read(float* u, const float* X, const float* a, int tokens, int S, int width, cudaStream_t s) {
    const size_t n = (size_t)tokens * width;
    if (!n) return;
    launch_k(streams_read_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, u, X, a, n, S, width);
    count_launch();
}
void streams_write(float* X, const float* y, const float* M, const float* b, int tokens, int S, int width, cudaStream_t s) {
    NT_CHECK(S >= 1 && S <= MAX_STREAMS, "streams_write: 1..16 streams");
    const size_t n = (size_t)tokens * width;
    if (!n) return;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (S == 1) launch_k(streams_write_kernel<1>, grid, dim3(256), 0, s, X, y, M, b, n, S, width);
    else if (S == 2) launch_k(streams_write_kernel<2>, grid, dim3(256), 0, s, X, y, M, b, n, S, width);
    else if (S == 3) launch_k(streams_write_kernel<3>, grid, dim3(256), 0, s, X, y, M, b, n, S, width);
    else if (S == 4) launch_k(streams_write_kernel<4>, grid, dim3(256), 0, s, X, y, M, b, n, S, width);
    else launch_k(streams_write_kernel<0>, grid, dim3(256), 0, s, X, y, M, b, n, S, width);
    count_launch();
}
void scale_rows(float* x, float scale, size_t n, cudaStream_t s) {
    if (!n) return;
    launch_k(scale_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, scale, n);
    count_launch();
}

}}  // namespace nt::b200
