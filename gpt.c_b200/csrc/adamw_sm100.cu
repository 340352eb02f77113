// AdamW step over a list of parameter tensors for sm_100a: one HBM-bound launch.
//
// Replaces step_adamW_cuda_kernel of gpt.c (kernels/src/cuda/AdamW.cu:64-148 and its kernel :13-57).  The
// reference uploads four pointer tables every step, synchronises the stream, and launches a grid sized for
// the largest tensor in which every thread walks all n tensors and skips the ones it is out of range for.
// Here the tables live on the device and are only re-uploaded when the host's tensor list changes, no
// synchronisation is needed, and the grid is a flat list of 4096-element chunks, each of which knows its
// tensor.  The arithmetic is the reference's, operation for operation (decoupled weight decay first, moments
// by the two-fma interpolation, bias corrections as multiplications).
#include <string.h>

#include <vector>

#include "attn_internal.h"
#include "tc05.cuh"

#include "../../include/adamw_sm100.h"

namespace adamw {
namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 4096;  // elements per block: four float4 per thread

struct Entry {
    float *p, *g, *m, *v;
    int len, pad;
};
struct Chunk {
    int tensor, start;
};

__device__ __forceinline__ float lerp_ref(float start, float end, float weight) {
    return fmaf(weight, end, fmaf(-weight, start, start));
}

__device__ __forceinline__ void update(float &p, float g, float &m, float &v, float lr, float beta1, float beta2, float wd,
                                       float eps, float c1, float c2) {
    p -= lr * wd * p;
    m = lerp_ref(g, m, beta1);
    v = lerp_ref(g * g, v, beta2);
    const float mh = m * c1, vh = v * c2;
    p -= lr * mh / (sqrtf(vh) + eps);
}

__global__ void __launch_bounds__(kThreads) adamw_kernel(const Entry *__restrict__ entries, const Chunk *__restrict__ chunks,
                                                         float lr, float beta1, float beta2, float wd, float eps, float c1,
                                                         float c2) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const Chunk ck = chunks[blockIdx.x];
    const Entry e = entries[ck.tensor];
    const int end = min(e.len, ck.start + kChunk);
    const bool vec = ((reinterpret_cast<uintptr_t>(e.p) | reinterpret_cast<uintptr_t>(e.g) | reinterpret_cast<uintptr_t>(e.m) |
                       reinterpret_cast<uintptr_t>(e.v)) & 15u) == 0;
    if (vec) {
        const int end4 = ck.start + ((end - ck.start) & ~3);
        for (int j = ck.start + 4 * threadIdx.x; j < end4; j += 4 * kThreads) {
            float4 p = *reinterpret_cast<float4 *>(e.p + j);
            const float4 g = __ldcs(reinterpret_cast<const float4 *>(e.g + j));
            float4 m = *reinterpret_cast<float4 *>(e.m + j);
            float4 v = *reinterpret_cast<float4 *>(e.v + j);
            update(p.x, g.x, m.x, v.x, lr, beta1, beta2, wd, eps, c1, c2);
            update(p.y, g.y, m.y, v.y, lr, beta1, beta2, wd, eps, c1, c2);
            update(p.z, g.z, m.z, v.z, lr, beta1, beta2, wd, eps, c1, c2);
            update(p.w, g.w, m.w, v.w, lr, beta1, beta2, wd, eps, c1, c2);
            *reinterpret_cast<float4 *>(e.p + j) = p;
            *reinterpret_cast<float4 *>(e.m + j) = m;
            *reinterpret_cast<float4 *>(e.v + j) = v;
        }
        for (int j = end4 + threadIdx.x; j < end; j += kThreads) update(e.p[j], e.g[j], e.m[j], e.v[j], lr, beta1, beta2, wd, eps, c1, c2);
    } else {
        for (int j = ck.start + threadIdx.x; j < end; j += kThreads) update(e.p[j], e.g[j], e.m[j], e.v[j], lr, beta1, beta2, wd, eps, c1, c2);
    }
}

// Device copies of the tensor list, per device, reused while the host list stays the same.
struct Cache {
    std::vector<Entry> host;
    Entry *d_entries = nullptr;
    Chunk *d_chunks = nullptr;
    size_t cap_entries = 0, cap_chunks = 0;
    int nchunks = 0;
};
Cache g_cache[64];

}  // namespace
}  // namespace adamw

extern "C" {

int adamw_sm100_step(float *const *params, float *const *grads, float *const *m, float *const *v, const int *lengths, int n,
                     float lr, float beta1, float beta2, float weight_decay, float eps, int step, void *stream) {
    using namespace adamw;
    if (!params || !grads || !m || !v || !lengths) return ATTN_ERR_NULL;
    if (n <= 0 || step <= 0) return ATTN_ERR_SHAPE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return ATTN_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Cache &c = g_cache[dev];

    std::vector<Entry> now((size_t)n);
    for (int i = 0; i < n; i++) {
        if (!params[i] || !grads[i] || !m[i] || !v[i]) return ATTN_ERR_NULL;
        if (lengths[i] < 0) return ATTN_ERR_SHAPE;
        now[i] = Entry{params[i], grads[i], m[i], v[i], lengths[i], 0};
    }
    const bool same = now.size() == c.host.size() && memcmp(now.data(), c.host.data(), now.size() * sizeof(Entry)) == 0;
    if (!same) {
        std::vector<Chunk> chunks;
        for (int i = 0; i < n; i++)
            for (int st = 0; st < lengths[i]; st += kChunk) chunks.push_back(Chunk{i, st});
        // the previous tables may still be in use by a launch in flight on this stream: stream-ordered free
        if (c.cap_entries < now.size()) {
            if (c.d_entries) cudaFreeAsync(c.d_entries, s);
            if ((e = cudaMallocAsync(reinterpret_cast<void **>(&c.d_entries), now.size() * sizeof(Entry), s)) != cudaSuccess) return (int)e;
            c.cap_entries = now.size();
        }
        if (c.cap_chunks < chunks.size()) {
            if (c.d_chunks) cudaFreeAsync(c.d_chunks, s);
            if ((e = cudaMallocAsync(reinterpret_cast<void **>(&c.d_chunks), chunks.size() * sizeof(Chunk), s)) != cudaSuccess) return (int)e;
            c.cap_chunks = chunks.size();
        }
        // pageable sources: the copies have read them by the time the calls return
        if ((e = cudaMemcpyAsync(c.d_entries, now.data(), now.size() * sizeof(Entry), cudaMemcpyHostToDevice, s)) != cudaSuccess) return (int)e;
        if (!chunks.empty() &&
            (e = cudaMemcpyAsync(c.d_chunks, chunks.data(), chunks.size() * sizeof(Chunk), cudaMemcpyHostToDevice, s)) != cudaSuccess)
            return (int)e;
        c.host = now;
        c.nchunks = (int)chunks.size();
    }
    if (c.nchunks == 0) return ATTN_OK;
    const float c1 = 1.0f / (1.0f - powf(beta1, (float)step));
    const float c2 = 1.0f / (1.0f - powf(beta2, (float)step));
    return (int)attn::launch_after_previous(adamw_kernel, dim3(c.nchunks), dim3(kThreads), 0, s, c.d_entries, c.d_chunks, lr, beta1,
                                            beta2, weight_decay, eps, c1, c2);
}

}  // extern "C"
