// attn_sm100_forward_static: the forward pass for callers that must not allocate.
//
// Some programs cannot give this library a scratch buffer and cannot let it call the CUDA
// allocator either: an inference server that handed all device memory to its own pool at
// start-up, a latency-critical loop where a cudaMalloc would stall the device, a host program
// whose rules forbid allocation after initialisation.  For them the bf16 hi/lo split of qkv (the
// `saved` buffer of attn_sm100_forward) lives in a fixed array inside the library image instead.
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine; the price is that
// every GPU that loads the library carries ATTN_STATIC_SCRATCH_BYTES of device memory until the
// process exits, and that larger problems are refused.
//
// The array is shared by all calls on a device and keeps whatever the last call left in it.  A
// call overwrites every byte it later reads, so nothing has to be cleared, but two calls that
// overlap on the GPU (different streams, different host threads) race on it.
#include "attn_internal.h"

#include <mutex>

#include "../../include/attn_sm100.h"

namespace {

// The split planes of one call: 2 planes x (B*T*3*H*D) bf16, each plane padded to 256 bytes.
static __device__ __align__(256) unsigned char g_static_scratch[ATTN_STATIC_SCRATCH_BYTES];
// Status word for bounded waits that run out inside the kernel (same meaning as the word read by
// attn_sm100_device_status, which belongs to the allocating path and is not touched here).
static __device__ int g_static_status;

constexpr int kMaxDevices = 64;
struct StaticState {
    bool ready = false;
    void *scratch = nullptr;  // DEVICE address of g_static_scratch on that device
    int *status = nullptr;
};
StaticState g_state[kMaxDevices];
std::mutex g_setup_lock;  // set-up is per device and may be entered by several host threads at once

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_static = nullptr;

// Once per device, with that device current.  In host code the names g_static_scratch and
// g_static_status are only stand-ins for the device objects: a kernel must be given the address
// cudaGetSymbolAddress returns, never &g_static_scratch itself.
int setup_device(int dev) {
    std::lock_guard<std::mutex> guard(g_setup_lock);
    StaticState &st = g_state[dev];
    if (st.ready) return ATTN_OK;
    int major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    if (major != 10) return ATTN_ERR_DEVICE;
    if (!g_encode_static) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return (int)e;
        if (q != cudaDriverEntryPointSuccess || !fn) return ATTN_ERR_DEVICE;
        g_encode_static = reinterpret_cast<EncodeTiledFn>(fn);
    }
    void *scratch = nullptr, *status = nullptr;
    e = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress(&status, g_static_status);
    if (e != cudaSuccess) return (int)e;
    if ((e = attn::fast_fwd_set_attributes()) != cudaSuccess) return (int)e;  // shared-memory opt-in, no allocation
    st.scratch = scratch;
    st.status = static_cast<int *>(status);
    st.ready = true;
    return ATTN_OK;
}

}  // namespace

extern "C" int attn_sm100_forward_static(const float *qkv, float *out, float *lse, int B, int T, int H, int D,
                                         void *stream) {
    if (!qkv || !out || !lse) return ATTN_ERR_NULL;
    if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return ATTN_ERR_SHAPE;
    if (D != 64) return ATTN_ERR_UNSUPPORTED;  // only the tensor-core forward needs (and has) this variant
    if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return ATTN_ERR_ALIGN;
    const double n_elems = (double)B * T * 3.0 * H * D;
    if (n_elems >= 2147483647.0) return ATTN_ERR_SHAPE;
    const size_t n = (size_t)B * T * 3 * H * D;
    const size_t plane = attn::plane_bytes(n);
    if (2 * plane > (size_t)ATTN_STATIC_SCRATCH_BYTES) return ATTN_ERR_STATIC_CAPACITY;

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return ATTN_ERR_DEVICE;
    int rc = setup_device(dev);  // first call on a device only; see the header about stream capture
    if (rc != ATTN_OK) return rc;
    const StaticState &st = g_state[dev];
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(st.scratch);
    __nv_bfloat16 *lo = reinterpret_cast<__nv_bfloat16 *>(static_cast<unsigned char *>(st.scratch) + plane);
    e = attn::launch_split(qkv, hi, lo, n, s);
    if (e != cudaSuccess) return (int)e;

    CUtensorMap map_x;
    const int W = 3 * H * D;
    const cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)T, (cuuint64_t)B, 2};
    const cuuint64_t strides[3] = {(cuuint64_t)W * 2, (cuuint64_t)W * 2 * (cuuint64_t)T, (cuuint64_t)plane};
    const cuuint32_t box[4] = {64, 64, 1, 1};  // the forward kernel loads 64-row boxes
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (g_encode_static(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, st.scratch, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return (int)cudaErrorInvalidValue;
    return (int)attn::launch_fast_forward(map_x, nullptr, nullptr, out, nullptr, lse, B, T, H, st.status, s);
}


// The status word of this entry point on the current device: the kernels above write it when a bounded
// wait runs out.  It is a word inside the library image, read and cleared with symbol copies, so this
// call allocates nothing either.
extern "C" int attn_sm100_static_status(int *status, int clear) {
    if (!status) return ATTN_ERR_NULL;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    e = cudaMemcpyFromSymbol(status, g_static_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_static_status, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return *status == 0 ? ATTN_OK : ATTN_ERR_KERNEL;
}
