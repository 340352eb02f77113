// Thin inline-PTX layer over the Blackwell (sm_100a) primitives the attention kernels use:
// mbarriers with bounded waits, TMA tiled loads, tensor-memory allocation, tcgen05 MMA issue,
// tensor-memory loads/stores, and the shared-memory / instruction descriptors of tcgen05.mma.
//
// Everything here is device-side and header-only.  No cluster-wide copy variants are used:
// every CTA issues its own loads from its own GPU's memory.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tc05 {

// ------------------------------------------------------------------------------------------
// Status words written by a kernel into the per-device status buffer when a bounded wait
// gives up.  0 means "no error".  The value encodes which wait ran out.
// ------------------------------------------------------------------------------------------
enum : int {
    ST_OK = 0,
    ST_TIMEOUT_BASE = 1000,  // ST_TIMEOUT_BASE + site id
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with launch_after_previous() (attn_internal.h) may
// start while the kernel before it in the stream is still running.  It must not touch global memory
// before pdl_wait() (returns once the previous kernel has completed and its writes are visible);
// pdl_launch_dependents() lets the kernel after this one start its own set-up.  Both are no-ops for a
// kernel launched the ordinary way.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of a barrier phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Shared abort word of a CTA plus the device-global status word.  A wait that runs out sets
// both; every later wait in the CTA returns false at once, so all roles fall through to the
// common tear-down (tensor memory is freed there) instead of spinning for ever.
struct WaitCtx {
    volatile int *cta_abort;  // shared memory
    int *status;              // global memory, may be nullptr
    uint64_t limit_ns;        // 0: TC05_WAIT_LIMIT_NS
};

#ifndef TC05_WAIT_LIMIT_NS
#define TC05_WAIT_LIMIT_NS 1000000000ull  // one second
#endif

// The part of a wait that is only reached when the first probe fails.  Not inlined: the kernels have
// dozens of waits, and the time-out logic repeated at each of them made their code a tenth larger.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, volatile int *cta_abort, int *status,
                                            uint64_t limit_ns, int site) {
    if (*cta_abort) return false;
    const uint64_t t0 = global_timer_ns();
    const uint64_t limit = limit_ns ? limit_ns : TC05_WAIT_LIMIT_NS;
    uint32_t it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++it & 63u) == 0u) {
            if (*cta_abort) return false;
            if (global_timer_ns() - t0 > limit) break;
        }
    }
    *cta_abort = 1;
    if (status) atomicCAS(status, 0, ST_TIMEOUT_BASE + site);
    return false;
}

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, const WaitCtx &ctx, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctx.cta_abort, ctx.status, ctx.limit_ns, site);
}

// Warp-uniform variant for warps that go on to execute .sync.aligned instructions: either every
// lane sees the barrier complete or the whole warp gives up together.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, const WaitCtx &ctx, int site) {
    const bool ok = mbar_wait(bar, parity, ctx, site);
    return __all_sync(0xffffffffu, ok);
}

// ------------------------------------------------------------------------------------------
// TMA: tiled loads global -> shared, completion signalled on an mbarrier (bytes).
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Shared -> global tile copies through a 3-D tensor map.  Rows outside the tensor are dropped.
// The copies of one thread form bulk groups: commit, then wait either until the shared-memory
// source has been read (the buffer may be rewritten) or until the group has completed.
__device__ __forceinline__ void tma_reduce_add_3d(const void *smem_src, const CUtensorMap *map, int c0, int c1, int c2) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void *smem_src, const CUtensorMap *map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// Tensor memory (TMEM) allocation.  Addresses are (lane << 16) | column.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // same warp as alloc
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ------------------------------------------------------------------------------------------
// Descriptors
// ------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, tile base 1024-byte aligned.
//   bits  0-13 start address >> 4        bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4   bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout type (2 = 128-byte swizzle)
// K-major operand  (rows of 128 bytes along K):  SBO = 1024 (next group of 8 rows), LBO unused.
// MN-major operand (rows of 128 bytes along M/N): SBO = 1024 (next group of 8 K-rows),
//                                                 LBO = distance between 64-element M/N blocks.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Advance the start address of a descriptor by `bytes` (must keep the 14-bit field in range).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
    return desc + (uint64_t)(bytes >> 4);
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   bit 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format (1 = bf16),
//   bit 15 A major (1 = MN), bit 16 B major (1 = MN), bits 17-22 N >> 3, bits 24-28 M >> 4.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ------------------------------------------------------------------------------------------
// MMA issue (one thread).  D[tmem] (+)= A * B;  K = 16 bf16 elements per instruction.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// A operand read from tensor memory (bf16 pairs packed in 32-bit columns, lane = row of A).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Warp-collective variants: the whole (converged) warp executes the call with identical operands
// and one elected lane issues the instruction.  Keeping the issuing loop warp-uniform lets the
// compiler hold descriptors in uniform registers instead of converting them per instruction.
__device__ __forceinline__ void mma_ss_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_commit_elect(uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}"
        ::"r"(smem_u32(bar))
        : "memory");
}

// The same with the election done once by the caller (elect_leader) for a whole batch of
// instructions: every MMA of a batch and the commit that tracks them are issued by one thread.
__device__ __forceinline__ uint32_t elect_leader() {
    uint32_t is_leader;
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, e;\n\t"
        "}"
        : "=r"(is_leader));
    return is_leader;
}

__device__ __forceinline__ void mma_ss_lead(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void mma_ts_lead(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

__device__ __forceinline__ void tc_commit_lead(uint32_t leader, uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "setp.ne.b32 e, %1, 0;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}"
        ::"r"(smem_u32(bar)), "r"(leader)
        : "memory");
}

// ------------------------------------------------------------------------------------------
// Tensor-memory loads / stores, shape 32x32b: lane t of the warp accesses TMEM lane
// (lane_base + t) and N consecutive 32-bit columns.  A warp may only touch the 32 lanes
// starting at 32 * (warp_id % 4).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ------------------------------------------------------------------------------------------
// bf16 hi/lo split: x ~= hi + lo with hi = bf16(x), lo = bf16(x - hi) (16 significant bits).
// Two values are packed per 32-bit word, the first argument in the low half.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo_half, float hi_half) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo_half, hi_half);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ void split_bf16x2(float a, float b, uint32_t &hi, uint32_t &lo) {
    hi = pack_bf16x2(a, b);
    const float ah = __uint_as_float(hi << 16);
    const float bh = __uint_as_float(hi & 0xFFFF0000u);
    lo = pack_bf16x2(a - ah, b - bh);
}

// ------------------------------------------------------------------------------------------
// Packed fp32 pairs (one instruction for two lanes of a float2) and 3-input max.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(*reinterpret_cast<unsigned long long *>(&d))
        : "l"(*reinterpret_cast<unsigned long long *>(&a)), "l"(*reinterpret_cast<unsigned long long *>(&b)),
          "l"(*reinterpret_cast<unsigned long long *>(&c)));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(*reinterpret_cast<unsigned long long *>(&d))
        : "l"(*reinterpret_cast<unsigned long long *>(&a)), "l"(*reinterpret_cast<unsigned long long *>(&b)));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(*reinterpret_cast<unsigned long long *>(&d))
        : "l"(*reinterpret_cast<unsigned long long *>(&a)), "l"(*reinterpret_cast<unsigned long long *>(&b)));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// hi/lo split of a pair with the residual computed as one packed fma: lo = bf16(p - float(hi)).
// The hi part is rounded to nearest (|p - hi| <= 2^-9 |p|).  Float-to-bf16 conversions run on the
// quarter-rate XU pipe together with exp2, which is the busiest pipe of the attention kernels, so
// the lo part is taken by truncation on the integer pipe instead (byte permute of the two upper
// halves): |p - hi - lo| < 2^-7 |p - hi| <= 2^-16 |p|.  TC05_SPLIT_MODE selects variants for
// experiments: 0 = both parts rounded, 1 = lo truncated (default), 2 = both truncated (2^-14).
#ifndef TC05_SPLIT_MODE
#define TC05_SPLIT_MODE 1
#endif
__device__ __forceinline__ void split_bf16x2_packed(float2 p, uint32_t &hi, uint32_t &lo) {
#if TC05_SPLIT_MODE == 2
    hi = __byte_perm(__float_as_uint(p.x), __float_as_uint(p.y), 0x7632);
    const float2 h = make_float2(__uint_as_float(__float_as_uint(p.x) & 0xFFFF0000u),
                                 __uint_as_float(__float_as_uint(p.y) & 0xFFFF0000u));
#else
    hi = pack_bf16x2(p.x, p.y);
    const float2 h = make_float2(__uint_as_float(hi << 16), __uint_as_float(hi & 0xFFFF0000u));
#endif
    const float2 r = fma2(h, make_float2(-1.f, -1.f), p);
#if TC05_SPLIT_MODE == 0
    lo = pack_bf16x2(r.x, r.y);
#else
    lo = __byte_perm(__float_as_uint(r.x), __float_as_uint(r.y), 0x7632);
#endif
}

}  // namespace tc05
