// C-ABI shim of libattn_sm100.so: argument validation, per-device set-up, tensor-map encoding
// and kernel dispatch.  Declarations and the reference interfaces they replace are in
// include/attn_sm100.h.
#include "attn_internal.h"
#include "tc05.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "../../include/attn_sm100.h"

namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
    std::atomic<bool> ready{false};  // set last, under g_init_lock; read without it on the fast path
    int *status = nullptr;  // device word written by kernels whose bounded waits run out
    int num_sms = 0;        // the persistent backward kernel runs one CTA per SM
};
DeviceState g_dev[kMaxDevices];
std::mutex g_init_lock;  // per-device set-up may be entered by several host threads at once

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

bool shape_ok(int B, int T, int H, int D) {
    if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return false;
    // element counts must fit the reference's 32-bit tensor_t.length (include/tensor.h:47)
    const double n = (double)B * T * 3.0 * H * D;
    return n < 2147483647.0;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool stages_ok(int flags) { return !((flags & ATTN_FLAG_PREPARE_ONLY) && (flags & ATTN_FLAG_CORE_ONLY)); }

bool use_fast(int D, int flags) { return D == 64 && !(flags & ATTN_FLAG_FORCE_GENERIC); }

// bf16 planes of a [B, T, W] tensor as a 4-D map {W, T, B, plane}, box {64, box_rows, 1, 1}.
int encode_planes(CUtensorMap *map, const void *base, int B, int T, int W, size_t plane_stride_bytes, int box_rows) {
    const cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)T, (cuuint64_t)B, 2};
    const cuuint64_t strides[3] = {(cuuint64_t)W * 2, (cuuint64_t)W * 2 * (cuuint64_t)T, (cuuint64_t)plane_stride_bytes};
    const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// fp32 [B, T, W] tensor as a 3-D map {W, T, B}, box {32, 128, 1}: the output side of the backward kernel.
int encode_rows_f32(CUtensorMap *map, const void *base, int B, int T, int W) {
    const cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)T, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)W * 4, (cuuint64_t)W * 4 * (cuuint64_t)T};
    const cuuint32_t box[3] = {32, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

int current_device_state(DeviceState **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ATTN_ERR_DEVICE;
    if (!g_dev[dev].ready.load(std::memory_order_acquire)) {
        const int rc = attn_sm100_init();
        if (rc != ATTN_OK) return rc;
    }
    *out = &g_dev[dev];
    return ATTN_OK;
}


// Exercises the bounded-wait path every tcgen05 kernel relies on, without touching the tensor
// cores: the barrier below is never completed, so the wait runs out after `limit_ns`, records
// ST_TIMEOUT_BASE + 900 in the status word and the kernel returns normally.
constexpr int kSelftestSite = 900;
__global__ void wait_limit_selftest_kernel(int *status, unsigned long long limit_ns) {
    __shared__ uint64_t never;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc05::mbar_init(&never, 1);
        tc05::fence_barrier_init();
    }
    __syncthreads();
    tc05::WaitCtx ctx{&abort_flag, status, limit_ns};
    tc05::mbar_wait_warp(&never, 0, ctx, kSelftestSite);
}

}  // namespace

namespace attn {

int encode_tiled(CUtensorMap *map, CUtensorMapDataType dtype, unsigned rank, const void *base, const cuuint64_t *dims,
                 const cuuint64_t *strides, const cuuint32_t *box, CUtensorMapSwizzle swizzle) {
    if (!g_encode) {
        const int rc = attn_sm100_init();
        if (rc != ATTN_OK) return rc;
    }
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = g_encode(map, dtype, rank, const_cast<void *>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

int device_status_word(int **status) {
    DeviceState *ds = nullptr;
    const int rc = current_device_state(&ds);
    if (rc != ATTN_OK) return rc;
    *status = ds->status;
    return ATTN_OK;
}

}  // namespace attn

extern "C" {

int attn_sm100_version(void) { return 100; }

int attn_sm100_init(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ATTN_ERR_DEVICE;
    if (g_dev[dev].ready.load(std::memory_order_acquire)) return ATTN_OK;
    std::lock_guard<std::mutex> guard(g_init_lock);
    if (g_dev[dev].ready.load(std::memory_order_relaxed)) return ATTN_OK;

    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    if (major != 10) return ATTN_ERR_DEVICE;

    if (!g_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return (int)e;
        if (q != cudaDriverEntryPointSuccess || !fn) return ATTN_ERR_DEVICE;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if ((e = attn::generic_set_attributes()) != cudaSuccess) return (int)e;
    if ((e = attn::fast_fwd_set_attributes()) != cudaSuccess) return (int)e;
    if ((e = attn::fast_bwd_set_attributes()) != cudaSuccess) return (int)e;

    int sms = 0;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    g_dev[dev].num_sms = sms;
    int *st = nullptr;
    if ((e = cudaMalloc(&st, sizeof(int))) != cudaSuccess) return (int)e;
    if ((e = cudaMemset(st, 0, sizeof(int))) != cudaSuccess) return (int)e;
    g_dev[dev].status = st;
    g_dev[dev].ready.store(true, std::memory_order_release);
    return ATTN_OK;
}

size_t attn_sm100_saved_bytes(int B, int T, int H, int D) {
    if (!shape_ok(B, T, H, D)) return 0;
    return 2 * attn::plane_bytes((size_t)B * T * 3 * H * D);
}

size_t attn_sm100_backward_scratch_bytes(int B, int T, int H, int D) {
    if (!shape_ok(B, T, H, D)) return 0;
    // dO planes, delta, and the two ints of the backward kernel's item counter
    return 2 * attn::plane_bytes((size_t)B * T * H * D) + attn::align_up((size_t)B * H * T * sizeof(float), 256) + 256;
}

int attn_sm100_forward(const float *qkv, float *out, float *out_copy, float *lse, void *saved, int B, int T, int H,
                       int D, int flags, void *stream) {
    if (!qkv || !out || !lse || !saved) return ATTN_ERR_NULL;
    if (!shape_ok(B, T, H, D) || !stages_ok(flags)) return ATTN_ERR_SHAPE;
    if (!aligned16(qkv) || !aligned16(out) || !aligned16(saved) || (out_copy && !aligned16(out_copy)))
        return ATTN_ERR_ALIGN;
    const bool fast = use_fast(D, flags);
    if (!fast && (D > attn::kGenericMaxD || T > attn::kGenericMaxT)) return ATTN_ERR_UNSUPPORTED;
    DeviceState *ds = nullptr;
    int rc = current_device_state(&ds);
    if (rc != ATTN_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const size_t n = (size_t)B * T * 3 * H * D;
    const size_t plane = attn::plane_bytes(n);
    __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(saved);
    __nv_bfloat16 *lo = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(saved) + plane);
    cudaError_t e = cudaSuccess;
    if (!(flags & ATTN_FLAG_CORE_ONLY)) {
        e = attn::launch_split(qkv, hi, lo, n, s);
        if (e != cudaSuccess) return (int)e;
    }
    if (flags & ATTN_FLAG_PREPARE_ONLY) return ATTN_OK;

    if (fast) {
        CUtensorMap map_x;
        rc = encode_planes(&map_x, saved, B, T, 3 * H * D, plane, 64);
        if (rc != 0) return rc;
        CUtensorMap map_out, map_copy;
        rc = encode_rows_f32(&map_out, out, B, T, H * D);
        if (rc != 0) return rc;
        if (out_copy) {
            rc = encode_rows_f32(&map_copy, out_copy, B, T, H * D);
            if (rc != 0) return rc;
        }
        e = attn::launch_fast_forward(map_x, &map_out, out_copy ? &map_copy : nullptr, out, out_copy, lse, B, T, H,
                                      ds->status, s);
    } else {
        e = attn::launch_generic_forward(qkv, out, out_copy, lse, B, T, H, D, s);
    }
    return (int)e;
}

int attn_sm100_backward(const void *saved, const float *out, const float *lse, const float *dout, float *dqkv,
                        void *scratch, int B, int T, int H, int D, int flags, void *stream) {
    if (!saved || !out || !lse || !dout || !dqkv || !scratch) return ATTN_ERR_NULL;
    if (!shape_ok(B, T, H, D) || !stages_ok(flags)) return ATTN_ERR_SHAPE;
    if (!aligned16(saved) || !aligned16(out) || !aligned16(dout) || !aligned16(dqkv) || !aligned16(scratch))
        return ATTN_ERR_ALIGN;
    const bool fast = use_fast(D, flags);
    if (!fast && (D > attn::kGenericMaxD || T > attn::kGenericMaxT)) return ATTN_ERR_UNSUPPORTED;
    DeviceState *ds = nullptr;
    int rc = current_device_state(&ds);
    if (rc != ATTN_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const size_t nx = (size_t)B * T * 3 * H * D, no = (size_t)B * T * H * D;
    const size_t xplane = attn::plane_bytes(nx), oplane = attn::plane_bytes(no);
    const __nv_bfloat16 *xhi = static_cast<const __nv_bfloat16 *>(saved);
    const __nv_bfloat16 *xlo = reinterpret_cast<const __nv_bfloat16 *>(static_cast<const char *>(saved) + xplane);
    __nv_bfloat16 *dhi = static_cast<__nv_bfloat16 *>(scratch);
    __nv_bfloat16 *dlo = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(scratch) + oplane);
    float *delta = reinterpret_cast<float *>(static_cast<char *>(scratch) + 2 * oplane);
    int *sched = reinterpret_cast<int *>(static_cast<char *>(scratch) + 2 * oplane +
                                         attn::align_up((size_t)B * H * T * sizeof(float), 256));

    cudaError_t e = cudaSuccess;
    const bool prepare = !(flags & ATTN_FLAG_CORE_ONLY), core = !(flags & ATTN_FLAG_PREPARE_ONLY);
    if (fast) {
        if (prepare) {
            e = attn::launch_bwd_prepare(dout, out, delta, dhi, dlo, dqkv, sched, B, T, H, D, s);
            if (e != cudaSuccess) return (int)e;
        }
        if (!core) return ATTN_OK;
        CUtensorMap map_x, map_do, map_dx;
        rc = encode_planes(&map_x, saved, B, T, 3 * H * D, xplane, 64);
        if (rc != 0) return rc;
        rc = encode_planes(&map_do, scratch, B, T, H * D, oplane, 64);
        if (rc != 0) return rc;
        rc = encode_rows_f32(&map_dx, dqkv, B, T, 3 * H * D);
        if (rc != 0) return rc;
        e = attn::launch_fast_backward(map_x, map_do, map_dx, lse, delta, dqkv, B, T, H, ds->num_sms, sched, ds->status, s);
    } else {
        if (prepare) {
            e = attn::launch_bwd_prepare(dout, out, delta, nullptr, nullptr, nullptr, nullptr, B, T, H, D, s);
            if (e != cudaSuccess) return (int)e;
        }
        if (!core) return ATTN_OK;
        e = attn::launch_generic_backward(xhi, xlo, lse, delta, dout, dqkv, B, T, H, D, s);
    }
    return (int)e;
}

int attn_sm100_selftest_wait_limit(unsigned limit_us, void *stream) {
    if (limit_us == 0 || limit_us > 100000u) return ATTN_ERR_SHAPE;  // at most 0.1 s
    DeviceState *ds = nullptr;
    const int rc = current_device_state(&ds);
    if (rc != ATTN_OK) return rc;
    wait_limit_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(ds->status, (unsigned long long)limit_us * 1000ull);
    return (int)cudaGetLastError();
}

int attn_sm100_device_status(int *status, int clear) {
    if (!status) return ATTN_ERR_NULL;
    DeviceState *ds = nullptr;
    int rc = current_device_state(&ds);
    if (rc != ATTN_OK) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    e = cudaMemcpy(status, ds->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (clear && *status != 0) {
        e = cudaMemset(ds->status, 0, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return *status == 0 ? ATTN_OK : ATTN_ERR_KERNEL;
}

const char *attn_sm100_strerror(int code) {
    switch (code) {
        case ATTN_OK: return "success";
        case ATTN_ERR_NULL: return "a required pointer is NULL";
        case ATTN_ERR_SHAPE: return "B, T, H and D must be positive and B*T*3*H*D must fit in 31 bits";
        case ATTN_ERR_UNSUPPORTED: return "shape not supported: head sizes other than 64 need D <= 256 and T <= 8192";
        case ATTN_ERR_ALIGN: return "pointers must be 16-byte aligned";
        case ATTN_ERR_DEVICE: return "the current device is not an sm_100 GPU or a driver entry point is missing";
        case ATTN_ERR_KERNEL: return "a kernel gave up a bounded wait (see attn_sm100_device_status)";
        case ATTN_ERR_STATIC_CAPACITY:
            return "attn_sm100_forward_static: B*T*3*H*D exceeds the 4,194,304 elements the built-in scratch array holds";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}

}  // extern "C"
