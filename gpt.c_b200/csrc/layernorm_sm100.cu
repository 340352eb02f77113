// LayerNorm forward and backward for sm_100a: HBM-bound row kernels.
//
// Replaces layer_norm_forward_cuda_kernel / layer_norm_backward_cuda_kernel of gpt.c
// (kernels/src/cuda/LayerNorm.cu:7-60 and :62-110: one 32-thread block per row, and in the backward
// one global atomicAdd per element for dW and db, i.e. rows x C atomics on C addresses).  Same
// arithmetic as the reference (mean and E[x^2] in one pass, rstd = 1/sqrt(var + eps); backward after
// the formulation the reference takes from PyTorch's CPU kernel, kernels/src/cpu/LayerNorm.c:96-121),
// same accumulate semantics: dW += , db += , dx += .
//
// One warp owns a row at a time and keeps it in registers (C <= 2048: up to 16 float4 per lane), so
// every tensor is read once.  In the backward each warp also carries the dW / db partial sums of its
// columns in registers over all the rows it visits; a block adds them up in shared memory and issues
// one atomicAdd per column, which cuts the atomics from rows x C to blocks x C.
#include <cooperative_groups.h>

#include "attn_internal.h"
#include "tc05.cuh"

#include "../../include/layernorm_sm100.h"

namespace ln {
namespace {

namespace cg = cooperative_groups;

constexpr int kWarpsPerBlock = 4;  // small blocks: the backward needs ~140 registers per thread at C = 768
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kCluster = 4;  // blocks whose column sums are combined before the atomics (backward)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// kNV: float4 chunks per lane, covering C <= 128 * kNV columns (C % 4 == 0)
template <int kNV>
__global__ void __launch_bounds__(kThreads) ln_forward_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                               const float *__restrict__ b, float eps,
                                                               float *__restrict__ mean, float *__restrict__ rstd,
                                                               float *__restrict__ y, int rows, int C) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * kWarpsPerBlock;
    const int nvec = C / 4;
    const float inv_c = 1.0f / (float)C;
    for (int row = warp; row < rows; row += nwarps) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * C);
        float4 v[kNV];
        float s = 0.f, ss = 0.f;
#pragma unroll
        for (int i = 0; i < kNV; i++) {
            const int c = lane + 32 * i;
            v[i] = c < nvec ? __ldcs(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += v[i].x + v[i].y + v[i].z + v[i].w;
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        s = warp_sum(s);
        ss = warp_sum(ss);
        const float m = s * inv_c;
        const float var = ss * inv_c - m * m;
        const float r = 1.0f / sqrtf(var + eps);
        float4 *yr = reinterpret_cast<float4 *>(y + (size_t)row * C);
#pragma unroll
        for (int i = 0; i < kNV; i++) {
            const int c = lane + 32 * i;
            if (c < nvec) {
                const float4 wv = __ldg(reinterpret_cast<const float4 *>(w) + c);
                float4 o;
                o.x = (v[i].x - m) * r * wv.x, o.y = (v[i].y - m) * r * wv.y;
                o.z = (v[i].z - m) * r * wv.z, o.w = (v[i].w - m) * r * wv.w;
                if (b) {
                    const float4 bv = __ldg(reinterpret_cast<const float4 *>(b) + c);
                    o.x += bv.x, o.y += bv.y, o.z += bv.z, o.w += bv.w;
                }
                yr[c] = o;
            }
        }
        if (lane == 0) {
            mean[row] = m;
            rstd[row] = r;
        }
    }
}

template <int kNV>
__global__ void __launch_bounds__(kThreads, (kNV <= 6 ? 4 : 1)) ln_backward_kernel(const float *__restrict__ dy, const float *__restrict__ x,
                                                                const float *__restrict__ mean,
                                                                const float *__restrict__ rstd, const float *__restrict__ w,
                                                                float *__restrict__ dw, float *__restrict__ db,
                                                                float *__restrict__ dx, int rows, int C) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    extern __shared__ float4 red[];  // [kWarpsPerBlock][nvec] partial sums, used twice (dW, then db), then [2][nvec]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int warp = blockIdx.x * kWarpsPerBlock + wid;
    const int nwarps = gridDim.x * kWarpsPerBlock;
    const int nvec = C / 4;
    const float inv_c = 1.0f / (float)C;
    float4 gw[kNV], gb[kNV];
#pragma unroll
    for (int i = 0; i < kNV; i++) {
        gw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        gb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float4 *w4 = reinterpret_cast<const float4 *>(w);  // re-read per row: it stays in L1
    for (int row = warp; row < rows; row += nwarps) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * C);
        const float4 *gr = reinterpret_cast<const float4 *>(dy + (size_t)row * C);
        const float a = rstd[row], mu = mean[row];
        const float nb = -a * mu;
        float4 *dr = reinterpret_cast<float4 *>(dx + (size_t)row * C);
        float4 xv[kNV], gv[kNV];
        // dx is accumulated into.  Fetching its old values together with x and dy (one trip to memory per row
        // instead of two) was measured and is no faster: it costs 40 registers, and the kernel is bound by how
        // many warps are in flight.
        constexpr bool kEarly = false;
        float4 ov[kEarly ? kNV : 1];
        float ds = 0.f, dbs = 0.f;
#pragma unroll
        for (int i = 0; i < kNV; i++) {
            const int c = lane + 32 * i;
            const bool in = c < nvec;
            xv[i] = in ? __ldcs(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            gv[i] = in ? __ldcs(gr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (kEarly) ov[i] = in ? dr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 wv = in ? __ldg(w4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            // from here on gv holds dy * w (what the input gradient needs); dy itself goes into the sums first
            gb[i].x += gv[i].x, gb[i].y += gv[i].y, gb[i].z += gv[i].z, gb[i].w += gv[i].w;
            gw[i].x += gv[i].x * (a * xv[i].x + nb), gw[i].y += gv[i].y * (a * xv[i].y + nb);
            gw[i].z += gv[i].z * (a * xv[i].z + nb), gw[i].w += gv[i].w * (a * xv[i].w + nb);
            gv[i].x *= wv.x, gv[i].y *= wv.y, gv[i].z *= wv.z, gv[i].w *= wv.w;
            ds += gv[i].x * xv[i].x + gv[i].y * xv[i].y + gv[i].z * xv[i].z + gv[i].w * xv[i].w;
            dbs += gv[i].x + gv[i].y + gv[i].z + gv[i].w;
        }
        ds = warp_sum(ds);
        dbs = warp_sum(dbs);
        const float bb = (dbs * mu - ds) * a * a * a * inv_c;
        const float cc = -bb * mu - dbs * a * inv_c;
#pragma unroll
        for (int i = 0; i < kNV; i++) {
            const int c = lane + 32 * i;
            if (c < nvec) {
                float4 o = kEarly ? ov[kEarly ? i : 0] : dr[c];  // accumulated, like the reference
                o.x += a * gv[i].x + bb * xv[i].x + cc, o.y += a * gv[i].y + bb * xv[i].y + cc;
                o.z += a * gv[i].z + bb * xv[i].z + cc, o.w += a * gv[i].w + bb * xv[i].w + cc;
                dr[c] = o;
            }
        }
    }
    // Column sums: over the warps of the block in shared memory, then over the kCluster blocks of the cluster
    // through distributed shared memory, then one atomic per column and cluster.  (With one atomic per column
    // and block, 444 blocks queued up on the same 1536 addresses and the kernel spent a third of its time
    // waiting for them to drain.)
    float4 *tot = red + kWarpsPerBlock * nvec;  // [2][nvec]: this block's sums for dW and db
    for (int pass = 0; pass < 2; pass++) {
#pragma unroll
        for (int i = 0; i < kNV; i++) {
            const int c = lane + 32 * i;
            if (c < nvec) red[wid * nvec + c] = pass == 0 ? gw[i] : gb[i];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < nvec; c += kThreads) {
            float4 t = red[c];
#pragma unroll
            for (int k = 1; k < kWarpsPerBlock; k++) {
                const float4 u = red[k * nvec + c];
                t.x += u.x, t.y += u.y, t.z += u.z, t.w += u.w;
            }
            tot[pass * nvec + c] = t;
        }
        __syncthreads();
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (cluster.block_rank() == 0) {
        for (int c = threadIdx.x; c < 2 * nvec; c += kThreads) {
            float *dst = c < nvec ? dw : db;
            if (dst == nullptr) continue;
            float4 t = tot[c];
            for (unsigned r = 1; r < cluster.num_blocks(); r++) {
                const float4 u = *cluster.map_shared_rank(tot + c, r);
                t.x += u.x, t.y += u.y, t.z += u.z, t.w += u.w;
            }
            const int col = 4 * (c < nvec ? c : c - nvec);
            atomicAdd(dst + col, t.x);
            atomicAdd(dst + col + 1, t.y);
            atomicAdd(dst + col + 2, t.z);
            atomicAdd(dst + col + 3, t.w);
        }
    }
    cluster.sync();  // the other blocks' shared memory stays alive until block 0 has read it
}

int grid_for(int rows, int blocks_per_sm) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = sms * blocks_per_sm;
    const int need = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    return grid < need ? grid : (need > 0 ? need : 1);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int kNV>
int launch_fwd(const float *x, const float *w, const float *b, float eps, float *mean, float *rstd, float *y, int rows, int C,
               cudaStream_t s) {
    return (int)attn::launch_after_previous(ln_forward_kernel<kNV>, dim3(grid_for(rows, 12)), dim3(kThreads), 0, s, x, w, b, eps,
                                            mean, rstd, y, rows, C);
}
template <int kNV>
int launch_bwd(const float *dy, const float *x, const float *mean, const float *rstd, const float *w, float *dw, float *db,
               float *dx, int rows, int C, cudaStream_t s) {
    const size_t smem = (size_t)(kWarpsPerBlock + 2) * (C / 4) * sizeof(float4);
    auto kernel = ln_backward_kernel<kNV>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // clusters of kCluster blocks (the grid is a whole number of them; blocks without rows add zeros),
    // launched as a programmatic dependent of the previous kernel like every kernel of the library
    const int grid = (grid_for(rows, kNV <= 6 ? 4 : 3) + kCluster - 1) / kCluster * kCluster;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = kCluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kernel, dy, x, mean, rstd, w, dw, db, dx, rows, C);
}

}  // namespace
}  // namespace ln

extern "C" {

int layernorm_sm100_forward(const float *x, const float *w, const float *b, float eps, float *mean, float *rstd, float *y,
                            int rows, int C, void *stream) {
    using namespace ln;
    if (!x || !w || !mean || !rstd || !y) return ATTN_ERR_NULL;
    if (rows <= 0 || C <= 0 || (long long)rows * C > 0x7fffffffLL) return ATTN_ERR_SHAPE;
    if (C % 4 != 0 || C > 2048) return ATTN_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(w) || !aligned16(b) || !aligned16(y)) return ATTN_ERR_ALIGN;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nv = (C + 127) / 128;
    if (nv <= 4) return launch_fwd<4>(x, w, b, eps, mean, rstd, y, rows, C, s);
    if (nv <= 6) return launch_fwd<6>(x, w, b, eps, mean, rstd, y, rows, C, s);
    if (nv <= 8) return launch_fwd<8>(x, w, b, eps, mean, rstd, y, rows, C, s);
    if (nv <= 10) return launch_fwd<10>(x, w, b, eps, mean, rstd, y, rows, C, s);
    if (nv <= 13) return launch_fwd<13>(x, w, b, eps, mean, rstd, y, rows, C, s);
    return launch_fwd<16>(x, w, b, eps, mean, rstd, y, rows, C, s);
}

int layernorm_sm100_backward(const float *dy, const float *x, const float *mean, const float *rstd, const float *w, float *dw,
                             float *db, float *dx, int rows, int C, void *stream) {
    using namespace ln;
    if (!dy || !x || !mean || !rstd || !w || !dw || !dx) return ATTN_ERR_NULL;
    if (rows <= 0 || C <= 0 || (long long)rows * C > 0x7fffffffLL) return ATTN_ERR_SHAPE;
    if (C % 4 != 0 || C > 2048) return ATTN_ERR_UNSUPPORTED;
    if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx)) return ATTN_ERR_ALIGN;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nv = (C + 127) / 128;
    if (nv <= 4) return launch_bwd<4>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
    if (nv <= 6) return launch_bwd<6>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
    if (nv <= 8) return launch_bwd<8>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
    if (nv <= 10) return launch_bwd<10>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
    if (nv <= 13) return launch_bwd<13>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
    return launch_bwd<16>(dy, x, mean, rstd, w, dw, db, dx, rows, C, s);
}

}  // extern "C"
