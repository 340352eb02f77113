// General-shape causal attention kernels (fp32 SIMT, one warp per row) and the elementwise
// preparation kernels shared with the tensor-core path.
//
// These kernels accept any head size D <= 256 and any T <= 8192.  They are the correctness
// anchor on the GPU and serve the shapes the tcgen05 kernels do not take (D != 64, e.g. the
// D = 3 case of the reference's tests/test_self_attention.py).  They replace the same
// reference code as the fast path: kernels/src/cuda/Attention.cu:170-324 of gpt.c.
#include "attn_internal.h"
#include "tc05.cuh"

namespace attn {

namespace {

constexpr int kWarp = 32;

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

// Element accessors: plain fp32, or the sum of the two bf16 planes written by the split kernel.
struct XF32 {
    const float *p;
    __device__ __forceinline__ float at(size_t i) const { return __ldg(p + i); }
};
struct XSplit {
    const __nv_bfloat16 *hi, *lo;
    __device__ __forceinline__ float at(size_t i) const {
        return __bfloat162float(hi[i]) + __bfloat162float(lo[i]);
    }
};

// ---------------------------------------------------------------------------------------
// split: x -> hi, lo
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) split_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ hi,
                                                     __nv_bfloat16 *__restrict__ lo, size_t n) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    const size_t n8 = n / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < n8; v += stride) {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(x) + 2 * v);
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(x) + 2 * v + 1);
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t h[4], l[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
            const float r0 = f[2 * k] - __low2float(hh), r1 = f[2 * k + 1] - __high2float(hh);
            __nv_bfloat162 ll = __floats2bfloat162_rn(r0, r1);
            h[k] = *reinterpret_cast<uint32_t *>(&hh);
            l[k] = *reinterpret_cast<uint32_t *>(&ll);
        }
        reinterpret_cast<uint4 *>(hi)[v] = make_uint4(h[0], h[1], h[2], h[3]);
        reinterpret_cast<uint4 *>(lo)[v] = make_uint4(l[0], l[1], l[2], l[3]);
    }
    // ragged tail (n not a multiple of 8)
    for (size_t i = n8 * 8 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float f = x[i];
        const __nv_bfloat16 hh = __float2bfloat16_rn(f);
        hi[i] = hh;
        lo[i] = __float2bfloat16_rn(f - __bfloat162float(hh));
    }
}

// ---------------------------------------------------------------------------------------
// backward preparation: delta[b,h,t] = sum_d dout*out, optional split of dout, optional
// zero-fill of the dq third of dqkv (the tensor-core backward accumulates dq with atomics).
// One warp per (b, t, h): D elements.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_prepare_kernel(const float *__restrict__ dout, const float *__restrict__ out,
                                                           float *__restrict__ delta, __nv_bfloat16 *__restrict__ dhi,
                                                           __nv_bfloat16 *__restrict__ dlo, float *__restrict__ dq_zero,
                                                           int B, int T, int H, int D) {
    const int lane = threadIdx.x & 31;
    const size_t nrows = (size_t)B * T * H;
    const size_t wstride = (size_t)gridDim.x * (blockDim.x >> 5);
    const int C = H * D;
    for (size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < nrows; w += wstride) {
        const int h = (int)(w % H);
        const size_t bt = w / H;
        const int t = (int)(bt % T);
        const int b = (int)(bt / T);
        const size_t base = bt * C + (size_t)h * D;
        float acc = 0.f;
        for (int d = lane; d < D; d += kWarp) {
            const float g = dout[base + d];
            acc += g * out[base + d];
            if (dhi) {
                const __nv_bfloat16 hh = __float2bfloat16_rn(g);
                dhi[base + d] = hh;
                dlo[base + d] = __float2bfloat16_rn(g - __bfloat162float(hh));
            }
            if (dq_zero) dq_zero[bt * 3 * C + (size_t)h * D + d] = 0.f;
        }
        acc = warp_sum(acc);
        if (lane == 0) delta[((size_t)b * H + h) * T + t] = acc;
    }
}

// ---------------------------------------------------------------------------------------
// backward preparation for head size 64 (the tensor-core path): the same work as above with
// 8 consecutive elements per thread, so 8 lanes cover one (b, t, h) row of 64 values.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_prepare64_kernel(const float *__restrict__ dout, const float *__restrict__ out,
                                                             float *__restrict__ delta, __nv_bfloat16 *__restrict__ dhi,
                                                             __nv_bfloat16 *__restrict__ dlo, float *__restrict__ dq_zero,
                                                             int *__restrict__ sched, int B, int T, int H) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    if (sched && blockIdx.x == 0 && threadIdx.x < 2) sched[threadIdx.x] = 0;  // item counter of the backward core
    const int C = H * 64;
    const size_t nvec = (size_t)B * T * C / 8;  // multiple of 8, so whole groups of 8 lanes stay together
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    // the loop bound is warp-uniform (shuffles below need every lane); memory accesses are guarded
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v - lane < nvec; v += stride) {
        const bool active = v < nvec;
        const size_t bt = v / (C / 8);
        const int c8 = (int)(v % (C / 8));
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 g0 = active ? __ldcs(reinterpret_cast<const float4 *>(dout) + 2 * v) : zero4;
        const float4 g1 = active ? __ldcs(reinterpret_cast<const float4 *>(dout) + 2 * v + 1) : zero4;
        const float4 o0 = active ? __ldcs(reinterpret_cast<const float4 *>(out) + 2 * v) : zero4;
        const float4 o1 = active ? __ldcs(reinterpret_cast<const float4 *>(out) + 2 * v + 1) : zero4;
        float acc = g0.x * o0.x + g0.y * o0.y + g0.z * o0.z + g0.w * o0.w + g1.x * o1.x + g1.y * o1.y + g1.z * o1.z +
                    g1.w * o1.w;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        const float f[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
            __nv_bfloat162 ll = __floats2bfloat162_rn(f[2 * k] - __low2float(hh), f[2 * k + 1] - __high2float(hh));
            hw[k] = *reinterpret_cast<uint32_t *>(&hh);
            lw[k] = *reinterpret_cast<uint32_t *>(&ll);
        }
        if (!active) continue;
        reinterpret_cast<uint4 *>(dhi)[v] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        reinterpret_cast<uint4 *>(dlo)[v] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        float4 *z = reinterpret_cast<float4 *>(dq_zero + bt * 3 * C + (size_t)c8 * 8);
        z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((c8 & 7) == 0) {
            const int h = c8 >> 3, t = (int)(bt % T), b = (int)(bt / T);
            delta[((size_t)b * H + h) * T + t] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------------
// generic forward: one warp per query row (b, h, i)
// shared memory per warp: T scores + D query values
// ---------------------------------------------------------------------------------------
template <class X>
__global__ void __launch_bounds__(128) generic_fwd_kernel(X x, float *__restrict__ out, float *__restrict__ out_copy,
                                                           float *__restrict__ lse, int B, int T, int H, int D,
                                                           float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nw = blockDim.x >> 5;
    const size_t row = (size_t)blockIdx.x * nw + warp;
    if (row >= (size_t)B * H * T) return;
    // longest rows first inside each (b, h)
    const int i = T - 1 - (int)(row % T);
    const size_t bh = row / T;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const int C = H * D, C3 = 3 * C;
    float *s = sm + (size_t)warp * (T + D);
    float *q = s + T;
    const size_t base = (size_t)b * T * C3;

    for (int d = lane; d < D; d += kWarp) q[d] = x.at(base + (size_t)i * C3 + (size_t)h * D + d);
    __syncwarp();

    float m = -INFINITY;
    for (int j = lane; j <= i; j += kWarp) {
        const size_t kp = base + (size_t)j * C3 + C + (size_t)h * D;
        float acc = 0.f;
        for (int d = 0; d < D; d++) acc = fmaf(q[d], x.at(kp + d), acc);
        acc *= scale;
        s[j] = acc;
        m = fmaxf(m, acc);
    }
    m = warp_max(m);
    float l = 0.f;
    for (int j = lane; j <= i; j += kWarp) {
        const float e = expf(s[j] - m);
        s[j] = e;
        l += e;
    }
    l = warp_sum(l);
    __syncwarp();
    const float inv = 1.0f / l;
    for (int d = lane; d < D; d += kWarp) {
        const size_t vp = base + 2 * (size_t)C + (size_t)h * D + d;
        float acc = 0.f;
        for (int j = 0; j <= i; j++) acc = fmaf(s[j], x.at(vp + (size_t)j * C3), acc);
        const size_t op = ((size_t)b * T + i) * C + (size_t)h * D + d;
        const float o = acc * inv;
        out[op] = o;
        if (out_copy) out_copy[op] = o;
    }
    if (lane == 0) lse[bh * T + i] = m + logf(l);
}

// ---------------------------------------------------------------------------------------
// generic backward, part 1: one warp per query row -> dq
// shared memory per warp: T values of dS + D (q) + D (dout row)
// ---------------------------------------------------------------------------------------
template <class X>
__global__ void __launch_bounds__(128) generic_bwd_dq_kernel(X x, const float *__restrict__ lse,
                                                              const float *__restrict__ delta,
                                                              const float *__restrict__ dout, float *__restrict__ dqkv,
                                                              int B, int T, int H, int D, float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nw = blockDim.x >> 5;
    const size_t row = (size_t)blockIdx.x * nw + warp;
    if (row >= (size_t)B * H * T) return;
    const int i = T - 1 - (int)(row % T);
    const size_t bh = row / T;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const int C = H * D, C3 = 3 * C;
    float *ds = sm + (size_t)warp * (T + 2 * D);
    float *q = ds + T;
    float *g = q + D;
    const size_t base = (size_t)b * T * C3;
    for (int d = lane; d < D; d += kWarp) {
        q[d] = x.at(base + (size_t)i * C3 + (size_t)h * D + d);
        g[d] = dout[((size_t)b * T + i) * C + (size_t)h * D + d];
    }
    __syncwarp();
    const float lse_i = lse[bh * T + i], delta_i = delta[bh * T + i];
    for (int j = lane; j <= i; j += kWarp) {
        const size_t kp = base + (size_t)j * C3 + C + (size_t)h * D;
        const size_t vp = kp + C;
        float sacc = 0.f, dp = 0.f;
        for (int d = 0; d < D; d++) {
            sacc = fmaf(q[d], x.at(kp + d), sacc);
            dp = fmaf(g[d], x.at(vp + d), dp);
        }
        const float p = expf(sacc * scale - lse_i);
        ds[j] = p * (dp - delta_i);
    }
    __syncwarp();
    for (int d = lane; d < D; d += kWarp) {
        const size_t kp = base + C + (size_t)h * D + d;
        float acc = 0.f;
        for (int j = 0; j <= i; j++) acc = fmaf(ds[j], x.at(kp + (size_t)j * C3), acc);
        dqkv[base + (size_t)i * C3 + (size_t)h * D + d] = acc * scale;
    }
}

// ---------------------------------------------------------------------------------------
// generic backward, part 2: one warp per key row -> dk, dv
// shared memory per warp: (T p values) + (T dS values) + D (k) + D (v)
// ---------------------------------------------------------------------------------------
template <class X>
__global__ void __launch_bounds__(128) generic_bwd_dkv_kernel(X x, const float *__restrict__ lse,
                                                               const float *__restrict__ delta,
                                                               const float *__restrict__ dout, float *__restrict__ dqkv,
                                                               int B, int T, int H, int D, float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nw = blockDim.x >> 5;
    const size_t row = (size_t)blockIdx.x * nw + warp;
    if (row >= (size_t)B * H * T) return;
    const int j = (int)(row % T);  // smallest j = longest column first
    const size_t bh = row / T;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const int C = H * D, C3 = 3 * C;
    float *ps = sm + (size_t)warp * (2 * T + 2 * D);
    float *dss = ps + T;
    float *kk = dss + T;
    float *vv = kk + D;
    const size_t base = (size_t)b * T * C3;
    for (int d = lane; d < D; d += kWarp) {
        kk[d] = x.at(base + (size_t)j * C3 + C + (size_t)h * D + d);
        vv[d] = x.at(base + (size_t)j * C3 + 2 * (size_t)C + (size_t)h * D + d);
    }
    __syncwarp();
    for (int i = j + lane; i < T; i += kWarp) {
        const size_t qp = base + (size_t)i * C3 + (size_t)h * D;
        const size_t gp = ((size_t)b * T + i) * C + (size_t)h * D;
        float sacc = 0.f, dp = 0.f;
        for (int d = 0; d < D; d++) {
            sacc = fmaf(x.at(qp + d), kk[d], sacc);
            dp = fmaf(dout[gp + d], vv[d], dp);
        }
        const float p = expf(sacc * scale - lse[bh * T + i]);
        ps[i - j] = p;
        dss[i - j] = p * (dp - delta[bh * T + i]);
    }
    __syncwarp();
    for (int d = lane; d < D; d += kWarp) {
        float dk = 0.f, dv = 0.f;
        for (int i = j; i < T; i++) {
            dk = fmaf(dss[i - j], x.at(base + (size_t)i * C3 + (size_t)h * D + d), dk);
            dv = fmaf(ps[i - j], dout[((size_t)b * T + i) * C + (size_t)h * D + d], dv);
        }
        dqkv[base + (size_t)j * C3 + C + (size_t)h * D + d] = dk * scale;
        dqkv[base + (size_t)j * C3 + 2 * (size_t)C + (size_t)h * D + d] = dv;
    }
}

int warps_for(size_t floats_per_warp) {
    const size_t bytes = floats_per_warp * sizeof(float);
    int nw = (int)(kGenericSmemLimit / bytes);
    return nw > 4 ? 4 : nw;
}

}  // namespace

cudaError_t generic_set_attributes() {
    cudaError_t e;
    e = cudaFuncSetAttribute(generic_fwd_kernel<XF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGenericSmemLimit);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(generic_bwd_dq_kernel<XSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kGenericSmemLimit);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(generic_bwd_dkv_kernel<XSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kGenericSmemLimit);
}

cudaError_t launch_split(const float *x, __nv_bfloat16 *hi, __nv_bfloat16 *lo, size_t n, cudaStream_t s) {
    const size_t work = (n + 7) / 8;
    size_t blocks = (work + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks == 0) blocks = 1;
    return launch_after_previous(split_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, hi, lo, n);
}

cudaError_t launch_bwd_prepare(const float *dout, const float *out, float *delta, __nv_bfloat16 *dhi,
                               __nv_bfloat16 *dlo, float *dq_zero, int *sched, int B, int T, int H, int D, cudaStream_t s) {
    if (D == 64 && dhi && dlo && dq_zero) {
        const size_t nvec = (size_t)B * T * H * 8;
        size_t blocks = (nvec + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        return launch_after_previous(bwd_prepare64_kernel, dim3((unsigned)blocks), dim3(256), 0, s, dout, out, delta, dhi,
                                     dlo, dq_zero, sched, B, T, H);
    }
    const size_t rows = (size_t)B * T * H;
    size_t blocks = (rows + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    bwd_prepare_kernel<<<(unsigned)blocks, 256, 0, s>>>(dout, out, delta, dhi, dlo, dq_zero, B, T, H, D);
    return cudaGetLastError();
}

cudaError_t launch_generic_forward(const float *qkv, float *out, float *out_copy, float *lse, int B, int T, int H,
                                   int D, cudaStream_t s) {
    const size_t per_warp = (size_t)T + D;
    const int nw = warps_for(per_warp);
    if (nw < 1) return cudaErrorInvalidValue;
    const size_t rows = (size_t)B * H * T;
    const size_t blocks = (rows + nw - 1) / nw;
    generic_fwd_kernel<XF32><<<(unsigned)blocks, nw * 32, nw * per_warp * sizeof(float), s>>>(
        XF32{qkv}, out, out_copy, lse, B, T, H, D, 1.0f / sqrtf((float)D));
    return cudaGetLastError();
}

cudaError_t launch_generic_backward(const __nv_bfloat16 *xhi, const __nv_bfloat16 *xlo, const float *lse,
                                    const float *delta, const float *dout, float *dqkv, int B, int T, int H, int D,
                                    cudaStream_t s) {
    const size_t rows = (size_t)B * H * T;
    const float scale = 1.0f / sqrtf((float)D);
    XSplit x{xhi, xlo};
    {
        const size_t per_warp = (size_t)T + 2 * D;
        const int nw = warps_for(per_warp);
        if (nw < 1) return cudaErrorInvalidValue;
        generic_bwd_dq_kernel<XSplit><<<(unsigned)((rows + nw - 1) / nw), nw * 32, nw * per_warp * sizeof(float), s>>>(
            x, lse, delta, dout, dqkv, B, T, H, D, scale);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    {
        const size_t per_warp = 2 * (size_t)T + 2 * D;
        const int nw = warps_for(per_warp);
        if (nw < 1) return cudaErrorInvalidValue;
        generic_bwd_dkv_kernel<XSplit><<<(unsigned)((rows + nw - 1) / nw), nw * 32, nw * per_warp * sizeof(float), s>>>(
            x, lse, delta, dout, dqkv, B, T, H, D, scale);
    }
    return cudaGetLastError();
}

}  // namespace attn
