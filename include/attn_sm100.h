/*
 * attn_sm100.h - C ABI of the Blackwell (sm_100a) causal self-attention library, libattn_sm100.so.
 *
 * The library replaces the CUDA attention path of gpt.c.  It computes, for the fused tensor
 * qkv [B, T, 3C] (C = H*D; q | k | v thirds, head h in columns h*D .. h*D+D-1 of each third),
 *
 *     out[b, i, h*D:(h+1)*D] = sum_{j<=i} softmax_j( q_i . k_j / sqrt(D) ) v_j          (forward)
 *     dqkv = [dq | dk | dv] for a given dout = dL/dout                                   (backward)
 *
 * in fp32 at the interface, without ever materialising the T x T score matrix.
 *
 * What each entry point stands in for in the reference (paths relative to the gpt.c root):
 *
 *   attn_sm100_init              runtime_init_cuda                 kernels/src/cuda/runtime.cu:16-29
 *   attn_sm100_forward           attention_forward_cuda_kernel     kernels/src/cuda/Attention.cu:170-232
 *                                (declared at kernels/src/cuda/Attention.h:9-15) together with the
 *                                permute/mask/softmax/unpermute kernels it launches (:12-75, :114-152,
 *                                kernels/src/cuda/Softmax.cu:7-76) and its two batched SGEMMs
 *                                (kernels/src/cuda/Tensor.cu:178-206)
 *   attn_sm100_backward          attention_backward_cuda_kernel    kernels/src/cuda/Attention.cu:235-324
 *                                (declared at kernels/src/cuda/Attention.h:17-22) with
 *                                kernels/src/cuda/Softmax.cu:78-119 and four batched SGEMMs
 *   attn_sm100_saved_bytes,      the cache allocations of forward_attention, src/attention.c:105-120
 *   attn_sm100_backward_scratch_bytes   and the temporaries of Attention.cu:256-258
 *   attn_sm100_device_status     cudaCheck(cudaGetLastError()) after each launch, e.g. Attention.cu:119
 *   attn_sm100_strerror          the CHECK_ERROR / cudaCheck message texts, include/utils.h:23,
 *                                kernels/src/cuda/cuda_common.h:61-68
 *
 * The reference passes tensor_t objects (include/tensor.h:44-51) and exits the process on error.
 * This ABI takes plain device pointers and sizes and returns a status instead, so the same entry
 * points serve the C layer (which maps non-zero to CHECK_ERROR), a ctypes harness and a
 * multi-GPU driver that shards the batch axis.
 *
 * Conventions
 *   - All pointers are device pointers on the CURRENT CUDA device; tensors are dense, row-major,
 *     and at least 16-byte aligned (cudaMalloc / cudaMallocAsync alignment is enough).
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *   - forward/backward only enqueue work: no allocation, no synchronisation, no host copies.
 *   - Return value: 0 on success, a negative ATTN_ERR_* for a rejected argument, or a positive
 *     cudaError_t when the CUDA runtime reported one.  Nothing is enqueued after an error.
 *   - There is no CPU fallback: every path is a CUDA kernel.
 *
 * Precision: operands are split into two bf16 terms (x ~ hi + lo, 16 significant bits) and each
 * product is evaluated as hi*hi + hi*lo + lo*hi on the tensor cores with fp32 accumulation;
 * softmax statistics are fp32.  Head sizes other than 64 take a general fp32 SIMT kernel.
 */
#ifndef ATTN_SM100_H
#define ATTN_SM100_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATTN_OK 0
#define ATTN_ERR_NULL (-1)        /* a required pointer is NULL */
#define ATTN_ERR_SHAPE (-2)       /* B, T, H or D is not positive, or an element count overflows */
#define ATTN_ERR_UNSUPPORTED (-3) /* shape outside what any kernel handles (see attn_sm100_forward) */
#define ATTN_ERR_ALIGN (-4)       /* a pointer is not 16-byte aligned */
#define ATTN_ERR_DEVICE (-5)      /* current device is not an sm_100 GPU, or a driver entry point is missing */
#define ATTN_ERR_KERNEL (-6)      /* reported by attn_sm100_device_status: a kernel gave up a bounded wait */
#define ATTN_ERR_STATIC_CAPACITY (-7) /* attn_sm100_forward_static: the problem needs more than ATTN_STATIC_SCRATCH_BYTES */

/* flags */
#define ATTN_FLAG_FORCE_GENERIC 1 /* use the general SIMT kernels even when the tensor-core path applies */
/* forward and backward each enqueue a preparation kernel (the bf16 hi/lo split of qkv; the split
 * of dout with rowsum(dout*out) and the zero-fill of dq) followed by the core attention kernel.
 * These two flags enqueue only one of the two stages, e.g. to time them separately or to reuse a
 * `saved` buffer that is already filled.  Setting both is an error (ATTN_ERR_SHAPE). */
#define ATTN_FLAG_PREPARE_ONLY 2
#define ATTN_FLAG_CORE_ONLY 4

/* Library version: major * 10000 + minor * 100 + patch. */
int attn_sm100_version(void);

/*
 * Prepares the current device: checks that it is compute capability 10.x, resolves the driver's
 * tensor-map encoder, raises the dynamic shared-memory limit of the kernels and allocates the
 * 4-byte device status word.  Idempotent; forward/backward call it on first use of a device, but
 * that first call allocates, so call it yourself before timing or capturing anything.
 */
int attn_sm100_init(void);

/*
 * Size in bytes of the `saved` buffer that forward fills and backward reads: the bf16 hi/lo
 * split of qkv, two planes of B*T*3C bf16 each, every plane padded to 256 bytes.
 * Returns 0 for an invalid shape.
 */
size_t attn_sm100_saved_bytes(int B, int T, int H, int D);

/*
 * Size in bytes of the scratch buffer backward needs (bf16 hi/lo split of dout, one fp32 per
 * (b, h, t) for rowsum(dout * out), and the counter from which the backward kernel's thread blocks
 * take their work items; the preparation stage of attn_sm100_backward initialises all of it).
 * Returns 0 for an invalid shape.
 */
size_t attn_sm100_backward_scratch_bytes(int B, int T, int H, int D);

/*
 * Forward.
 *   qkv      [B, T, 3*H*D] fp32, read only
 *   out      [B, T, H*D]   fp32, written
 *   out_copy [B, T, H*D]   fp32, written with the same values when not NULL (the layer keeps it
 *                          for backward because the caller's `out` is consumed by the next layer)
 *   lse      [B, H, T]     fp32, written: log(sum_j exp(s_ij)) of the scaled scores
 *   saved    attn_sm100_saved_bytes() bytes, written; must stay intact until backward has run
 * D == 64 runs the tcgen05 tensor-core kernel for any T >= 1.  Other D run the general kernel,
 * which needs D <= 256 and T <= 8192; larger values return ATTN_ERR_UNSUPPORTED.
 */
int attn_sm100_forward(const float *qkv, float *out, float *out_copy, float *lse, void *saved,
                       int B, int T, int H, int D, int flags, void *stream);

/*
 * Backward.
 *   saved    what forward wrote for the same qkv
 *   out, lse what forward wrote (out may be the out_copy)
 *   dout     [B, T, H*D]   fp32, read only
 *   dqkv     [B, T, 3*H*D] fp32, every element written ([dq | dk | dv] per token); it does not
 *                          need to be zeroed by the caller
 *   scratch  attn_sm100_backward_scratch_bytes() bytes, clobbered
 */
int attn_sm100_backward(const void *saved, const float *out, const float *lse, const float *dout,
                        float *dqkv, void *scratch, int B, int T, int H, int D, int flags, void *stream);

/*
 * Forward without any allocation.  (No counterpart in the reference: gpt.c allocates its caches with
 * cudaMallocAsync on every call, kernels/src/cuda/Alloc.cu:9-14.)
 *
 * For callers that can neither pass a scratch buffer nor let the library enter the CUDA allocator:
 * a server whose own pool owns all device memory, a latency-critical loop that must not risk the
 * device-wide stall of a cudaMalloc, a host with a no-allocation-after-start-up rule.  The bf16 hi/lo
 * split of qkv is kept in a fixed device array inside the library (ATTN_STATIC_SCRATCH_BYTES, held by
 * every GPU that loads the library until the process exits) instead of a `saved` buffer, so the call
 * is forward-only: there is nothing to hand to attn_sm100_backward.
 *   qkv [B, T, 3*H*64] fp32 in, out [B, T, H*64] fp32, lse [B, H, T] fp32; D must be 64.
 * Limits and rules
 *   - 4 * B*T*3*H*D bytes (two bf16 planes, each padded to 256) must fit in ATTN_STATIC_SCRATCH_BYTES,
 *     i.e. B*T*3*H*D <= 4,194,304 elements; larger problems return ATTN_ERR_STATIC_CAPACITY.
 *   - No cudaMalloc / cudaFree / allocating library call is made, not even on first use.  The first
 *     call on each device resolves the device address of the array (cudaGetSymbolAddress) and raises
 *     the kernel's shared-memory limit.  With CUDA's lazy module loading that first call is also the
 *     moment the driver loads this library's code onto the device and reserves the array there, which
 *     can take as long as an allocation: make the first call per device at start-up, and before
 *     starting any stream capture.
 *   - All calls on a device share the array and it keeps the previous call's contents.  Each call
 *     rewrites every byte it reads, so nothing needs clearing, but calls that overlap on the GPU
 *     (other streams or threads) race on it: serialise them.
 *   - Kernel status for this path is separate from attn_sm100_device_status: read it with
 *     attn_sm100_static_status.
 */
#define ATTN_STATIC_SCRATCH_BYTES (16u << 20)
int attn_sm100_forward_static(const float *qkv, float *out, float *lse, int B, int T, int H, int D, void *stream);

/*
 * Status word of attn_sm100_forward_static on the current device (no counterpart in the reference).
 * Synchronises the device; *status receives 0, or a code >= 1000 naming the bounded wait that ran out
 * inside a kernel launched by attn_sm100_forward_static (its out / lse are then not valid).  When `clear`
 * is non-zero the word is reset.  The word lives inside the library image like the scratch array, so this
 * call allocates nothing.  Returns ATTN_OK, ATTN_ERR_KERNEL when *status != 0, or a cudaError_t.
 */
int attn_sm100_static_status(int *status, int clear);

/*
 * Failure-path self-test (no counterpart in the reference, which has no bounded waits): launches a
 * one-CTA kernel that waits, with the same helper every tcgen05 kernel of this library uses, on a
 * barrier that is never completed.  After `limit_us` microseconds (1..100000) the wait gives up,
 * the kernel returns normally and the device status word holds 1900; attn_sm100_device_status then
 * returns ATTN_ERR_KERNEL until the word is cleared.  Nothing faults, traps or spins for ever, and
 * the context stays usable.  Returns ATTN_OK when the kernel was enqueued, ATTN_ERR_SHAPE for a
 * limit outside the range, or a cudaError_t.
 */
int attn_sm100_selftest_wait_limit(unsigned limit_us, void *stream);

/*
 * Synchronises the current device and reads its status word.  *status receives 0, or a code
 * >= 1000 naming the bounded wait that ran out inside a kernel.  When `clear` is non-zero the
 * word is reset.  Returns ATTN_OK, ATTN_ERR_KERNEL when *status != 0, or a cudaError_t.
 */
int attn_sm100_device_status(int *status, int clear);

/* Human-readable text for a return value of this library (static storage). */
const char *attn_sm100_strerror(int code);

#ifdef __cplusplus
}
#endif

#endif /* ATTN_SM100_H */
