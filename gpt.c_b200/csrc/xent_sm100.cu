// Cross-entropy loss over the vocabulary for sm_100a: HBM-bound row kernels.
//
// Replaces cross_entropy_forward_cuda_kernel / cross_entropy_backward_cuda_kernel of gpt.c
// (kernels/src/cuda/CrossEntropyLoss.cu:136-178 and their kernels :8-79, :82-129: one warp per row of
// 50257 logits, three passes forward).  Same results and the same buffer semantics:
//   forward   logsm[r, :] = logits[r, :] - max - log(sum exp(logits - max));  loss += -logsm[r, target_r] / rows
//   backward  dout[r, target_r] = -g[r] / rows;  s = sum_j dout[r, j];  dout[r, j] -= exp(logsm[r, j]) * s
// (the backward works on whatever dout holds, like the reference, whose layer hands in zeros).
//
// One block of 1024 threads per row; the rows of a [rows, 50257] tensor start on 4-byte boundaries only,
// so loads and stores are 4 bytes wide but fully coalesced.  Forward: maximum and sum of exponentials in
// one online pass, then the write pass re-reads the row (200 KB): 8 bytes of HBM traffic per element when the
// re-read hits L2.  The forward loops keep eight loads per thread in flight: with one load per trip, which is
// what the dependent maximum / sum update compiles to, the pass was bound by memory latency, not bandwidth.
// (The backward loops have independent trips and gained nothing from the same change.)
// Backward: 12 bytes per element (dout is read-modify-write; its second read hits L2 the same way).
#include "attn_internal.h"
#include "tc05.cuh"

#include "../../include/xent_sm100.h"

namespace xent {
namespace {

constexpr int kThreads = 1024;
constexpr int kBatch = 8;  // independent loads per thread and loop trip

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kThreads) xent_forward_kernel(const float *__restrict__ logits,
                                                                const float *__restrict__ targets,
                                                                float *__restrict__ logsm, float *__restrict__ loss,
                                                                int rows, int C) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    __shared__ float s_m[kThreads / 32], s_s[kThreads / 32];
    __shared__ float s_shift;
    const int r = blockIdx.x;
    const float *x = logits + (size_t)r * C;
    float *y = logsm + (size_t)r * C;
    // online maximum / sum of exponentials
    float m = -INFINITY, s = 0.f;
    for (int j0 = threadIdx.x; j0 < C; j0 += kThreads * kBatch) {
        float v[kBatch];  // kBatch loads in flight per thread: the pass is bound by HBM latency otherwise
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int j = j0 + u * kThreads;
            v[u] = j < C ? __ldg(x + j) : -INFINITY;
        }
        float bm = v[0];
#pragma unroll
        for (int u = 1; u < kBatch; u++) bm = fmaxf(bm, v[u]);
        if (bm > m) {
            s *= __expf(m - bm);  // exp(-inf) = 0 on the first batch
            m = bm;
        }
#pragma unroll
        for (int u = 0; u < kBatch; u++) s += __expf(v[u] - m);  // exp(-inf) = 0 past the end of the row
    }
    // combine (m, s) pairs across the warp, then across the block
    const float wm = warp_max(m);
    s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
    if ((threadIdx.x & 31) == 0) {
        s_m[threadIdx.x >> 5] = wm;
        s_s[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const float pm = threadIdx.x < kThreads / 32 ? s_m[threadIdx.x] : -INFINITY;
        const float ps = threadIdx.x < kThreads / 32 ? s_s[threadIdx.x] : 0.f;
        const float bm = warp_max(pm);
        const float bs = warp_sum(pm == -INFINITY ? 0.f : ps * __expf(pm - bm));
        if (threadIdx.x == 0) s_shift = bm + logf(bs);
    }
    __syncthreads();
    const float shift = s_shift;
    for (int j0 = threadIdx.x; j0 < C; j0 += kThreads * kBatch) {
        float v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int j = j0 + u * kThreads;
            v[u] = j < C ? __ldg(x + j) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int j = j0 + u * kThreads;
            if (j < C) y[j] = v[u] - shift;
        }
    }
    if (threadIdx.x == 0) {
        const int t = (int)targets[r];
        atomicAdd(loss, -(x[t] - shift) / (float)rows);
    }
}

__global__ void __launch_bounds__(kThreads) xent_backward_kernel(const float *__restrict__ g,
                                                                 const float *__restrict__ targets,
                                                                 const float *__restrict__ logsm, float *__restrict__ dout,
                                                                 int rows, int C) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    __shared__ float s_part[kThreads / 32];
    __shared__ float s_total;
    const int r = blockIdx.x;
    const float *c = logsm + (size_t)r * C;
    float *d = dout + (size_t)r * C;
    const int t = (int)targets[r];
    const float at_target = -g[r] / (float)rows;
    // sum of the row as it will be once the target entry is set
    float s = 0.f;
    for (int j = threadIdx.x; j < C; j += kThreads) s += j == t ? at_target : d[j];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float p = threadIdx.x < kThreads / 32 ? s_part[threadIdx.x] : 0.f;
        p = warp_sum(p);
        if (threadIdx.x == 0) s_total = p;
    }
    __syncthreads();
    const float total = s_total;
    for (int j = threadIdx.x; j < C; j += kThreads) {
        const float cur = j == t ? at_target : d[j];
        d[j] = cur - __expf(c[j]) * total;
    }
}

}  // namespace
}  // namespace xent

extern "C" {

int xent_sm100_forward(const float *logits, const float *targets, float *logsm, float *loss, int rows, int C, void *stream) {
    if (!logits || !targets || !logsm || !loss) return ATTN_ERR_NULL;
    if (rows <= 0 || C <= 0) return ATTN_ERR_SHAPE;
    return (int)attn::launch_after_previous(xent::xent_forward_kernel, dim3(rows), dim3(xent::kThreads), 0,
                                            static_cast<cudaStream_t>(stream), logits, targets, logsm, loss, rows, C);
}

int xent_sm100_backward(const float *g, const float *targets, const float *logsm, float *dout, int rows, int C, void *stream) {
    if (!g || !targets || !logsm || !dout) return ATTN_ERR_NULL;
    if (rows <= 0 || C <= 0) return ATTN_ERR_SHAPE;
    return (int)attn::launch_after_previous(xent::xent_backward_kernel, dim3(rows), dim3(xent::kThreads), 0,
                                            static_cast<cudaStream_t>(stream), g, targets, logsm, dout, rows, C);
}

}  // extern "C"
