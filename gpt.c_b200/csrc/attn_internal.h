// Internal launch interface between the C-ABI shim (attn_api.cu) and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace attn {

constexpr int kGenericMaxD = 256;
constexpr int kGenericMaxT = 8192;
constexpr int kGenericSmemLimit = 200 * 1024;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// One bf16 plane of n elements, padded so the next plane starts 256-byte aligned.
inline size_t plane_bytes(size_t n) { return align_up(n * sizeof(__nv_bfloat16), 256); }

// fp32 -> (hi, lo) bf16 planes, hi = bf16(x), lo = bf16(x - hi).
cudaError_t launch_split(const float *x, __nv_bfloat16 *hi, __nv_bfloat16 *lo, size_t n, cudaStream_t s);

// rowsum(dout * out) per (b, h, t) -> delta [B, H, T]; also splits dout into bf16 planes when
// dhi/dlo are given, zero-fills the dq third of `dq_zero` ([B, T, 3C]) when it is given, and zeroes the
// two ints at `sched` (the item counter of the tensor-core backward kernel) when that is given.
cudaError_t launch_bwd_prepare(const float *dout, const float *out, float *delta, __nv_bfloat16 *dhi,
                               __nv_bfloat16 *dlo, float *dq_zero, int *sched, int B, int T, int H, int D, cudaStream_t s);

// General-shape SIMT kernels (any D <= kGenericMaxD, T <= kGenericMaxT).
cudaError_t generic_set_attributes();
cudaError_t launch_generic_forward(const float *qkv, float *out, float *out_copy, float *lse, int B, int T, int H,
                                   int D, cudaStream_t s);
cudaError_t launch_generic_backward(const __nv_bfloat16 *xhi, const __nv_bfloat16 *xlo, const float *lse,
                                    const float *delta, const float *dout, float *dqkv, int B, int T, int H, int D,
                                    cudaStream_t s);

// Tensor-core (tcgen05) kernels, D == 64.  The tensor maps cover the bf16 hi/lo planes:
//   map_x : dims {3C, T, B, 2 planes}, box {64, 128, 1, 1}, 128-byte swizzle
//   map_do: dims { C, T, B, 2 planes}, same box
cudaError_t fast_fwd_set_attributes();
cudaError_t fast_bwd_set_attributes();
cudaError_t launch_fast_forward(const CUtensorMap &map_x, const CUtensorMap *map_out, const CUtensorMap *map_copy,
                                float *out, float *out_copy, float *lse, int B, int T, int H, int *status, cudaStream_t s);
cudaError_t launch_fast_backward(const CUtensorMap &map_x, const CUtensorMap &map_do, const CUtensorMap &map_dx,
                                 const float *lse, const float *delta, float *dqkv, int B, int T, int H, int num_sms,
                                 int *sched, int *status, cudaStream_t s);

// Launches `kernel` so that it may begin (up to its pdl_wait(), tc05.cuh) while the previous kernel of the
// stream is still running: its launch latency and set-up overlap that kernel's tail.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_previous(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                         Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Helpers shared with the Linear kernels (linear_sm100.cu).
// cuTensorMapEncodeTiled with the given swizzle, no interleave, no L2 promotion, zero fill; the encoder
// is resolved by attn_sm100_init.  Returns 0 or a cudaError_t.
int encode_tiled(CUtensorMap *map, CUtensorMapDataType dtype, unsigned rank, const void *base, const cuuint64_t *dims,
                 const cuuint64_t *strides, const cuuint32_t *box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);
// Status word of the current device (initialises the library on first use).  Returns ATTN_OK or an error.
int device_status_word(int **status);

}  // namespace attn
