// Linear layer (y = x W^T + b) and its backward for sm_100a: one persistent tcgen05 GEMM kernel
// with TF32 inputs read straight from the fp32 tensors and fp32 accumulation in tensor memory.
//
// Replaces linear_forward_cuda_kernel / linear_backward_cuda_kernel of gpt.c
// (kernels/src/cuda/Linear.cu:37-92: one cuBLAS SGEMM in TF32 tensor-op math plus a separate
// bias kernel forward; two SGEMMs plus an atomic bias reduction backward) for the two Linear
// layers either side of the attention layer (src/self_attention.c:59-61, 78-80).  The forward
// epilogue adds the bias and can also emit the result as the two bf16 planes (hi, lo) the
// attention kernels consume, which removes the attention path's own split pass.
//
// The three products differ only in which operand dimension is contiguous in memory:
//     forward  y [M,N]  = x [M,K] . W[N,K]^T        A: x, K-major          B: W,  K-major
//     dx       dx[M,K]  = dy[M,N] . W[N,K]          A: dy, K-major (over N) B: W,  MN-major
//     dW       dW[N,K] += dy[M,N]^T . x[M,K]        A: dy, MN-major         B: x,  MN-major  (split over M)
// (K-major: the contraction index is the contiguous one.)  Tiles are 128 x 128 with contraction
// blocks of 32 fp32 values (one 128-byte swizzled row), four stages.
//
// Warp roles (384 threads, one CTA per SM, grid = number of SMs, tiles handed out round robin):
//   warp 0      TMA producer
//   warp 1      MMA issuer (kind::tf32, M128 N128 K8, one elected lane)
//   warp 2      tensor-memory allocation (2 accumulators of 128 columns: the epilogue of one tile
//               overlaps the main loop of the next)
//   warps 4-11  epilogue, two warps per tensor-memory lane quarter: accumulator -> registers ->
//               (+bias, bf16 split) -> swizzled staging tile in shared memory
//   warp 3      bulk tensor store (forward, dx) or bulk tensor reduction (dW) of each staged chunk
// All waits are bounded (see tc05.cuh).
#include "attn_internal.h"
#include "tc05.cuh"

#include "../../include/linear_sm100.h"
#include "../../include/tensor_sm100.h"

namespace lin {
namespace {

using namespace tc05;

constexpr int kBM = 128, kBK = 32;
constexpr int kATileBytes = kBM * kBK * 4;  // A tile of one stage: 16 KiB
constexpr int kThreads = 384;
constexpr int kEpiThreads = 256;

// Tile width kBN (128 or 256 columns) and pipeline depth are chosen per problem: wide tiles halve the
// shared-memory and L2 traffic per flop, narrow ones fill the SMs better when there are few tiles.
template <int kBN, int kStages, bool kPlanes>
struct __align__(1024) SmemT {
    uint8_t a[kStages][kATileBytes];
    uint8_t b[kStages][kBN * kBK * 4];
    // 64 output columns of a tile on their way out: fp32 columns 0-31 and fp32 columns 32-63; when the bf16
    // planes are wanted, the same two buffers then carry the hi plane (64 columns) and the lo plane of the
    // chunk (a second round through the copy engine: two more buffers would cost a pipeline stage, and the
    // depth of the operand pipeline is what bounds this kernel); each [128 rows x 128 bytes], swizzled
    // 192-wide tiles without planes stage through ONE buffer (32 columns per round): that leaves room for a
    // fifth pipeline stage of 40 KB
    uint8_t out[(kBN == 192 && !kPlanes) ? 1 : 2][16384];
    uint64_t full[kStages], empty[kStages];
    uint64_t acc_full[2], acc_empty[2];
    uint64_t out_ready, out_free;
    uint32_t tmem_base;
    int abort_flag;
};

struct Problem {
    int M, N, K;  // C is [M, N]; K is the contraction length
    int bn;       // tile width
    int a_one, b_one;  // MN-major operand fetched with one 3-D copy per stage (else one copy per 32-row block)
    int tiles_m, tiles_n, splits, kb_total, kb_per_split, total;
    int m_fast;  // consecutive work items walk down the rows of C (else along its columns)
};

enum Site : int {
    SITE_EMPTY = 201, SITE_FULL, SITE_ACC_EMPTY, SITE_ACC_FULL, SITE_OUT_READY, SITE_OUT_FREE, SITE_SMEM_ALIGN
};

// Instruction descriptor for kind::tf32 (A and B formats = 2), fp32 accumulation.
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32_lead(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 e, %5, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}

// Shared-memory descriptor for 32-bit operands read MN-major: layout type 1 (128-byte swizzle with
// 32-byte atoms); rows of 32 values along M/N, LBO = distance between 32-value blocks, SBO = distance
// between groups of 4 contraction steps.
__device__ __forceinline__ uint64_t smem_desc_sw128_base32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

struct Work {
    int m0, n0, kb0, kb1;
};
__device__ __forceinline__ Work decode(const Problem &p, int w) {
    const int split = w % p.splits;
    const int t = w / p.splits;
    // The operand whose tile index changes slowest is read from HBM once; the other one is streamed again for
    // every step of the slow index and has to live in L2.  The host picks the order by operand size.
    const int tn = p.m_fast ? t / p.tiles_m : t % p.tiles_n;
    const int tm = p.m_fast ? t % p.tiles_m : t / p.tiles_n;
    Work r;
    r.m0 = tm * kBM;
    r.n0 = tn * p.bn;
    r.kb0 = split * p.kb_per_split;
    r.kb1 = min(p.kb_total, r.kb0 + p.kb_per_split);
    return r;
}

// kEpi 0: C = acc (+ bias), optional bf16 planes; kEpi 1: C += acc (bulk reduction)
// kDirect: the result goes out with plain coalesced 4-byte stores instead of the copy engine, for outputs
// whose row pitch is not a multiple of 16 bytes (the 50257-wide vocabulary projection).
template <bool kAMN, bool kBMN, int kEpi, int kBN, int kStages, bool kPlanes, bool kDirect = false>
__global__ void __launch_bounds__(kThreads, 1)
linear_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_planes,
                   const float *__restrict__ bias, float *__restrict__ c_direct, Problem p, int *status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    using Smem = SmemT<kBN, kStages, kPlanes>;
    constexpr uint32_t kTmemCols = 2 * kBN <= 256 ? 256 : 512;  // a power of two that holds two accumulators
    constexpr int kBTileBytes = kBN * kBK * 4;
    constexpr bool kOut1 = kBN == 192 && !kPlanes;  // one output staging buffer (see SmemT)
    Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_TIMEOUT_BASE + SITE_SMEM_ALIGN);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    WaitCtx ctx{&sm.abort_flag, status};
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        for (int i = 0; i < kStages; i++) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm.acc_full[i], 1);
            mbar_init(&sm.acc_empty[i], kEpiThreads);
        }
        mbar_init(&sm.out_ready, kEpiThreads);
        mbar_init(&sm.out_free, kDirect ? kEpiThreads : 1);
        fence_barrier_init();
    }
    if (warp == 2) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    pdl_wait();  // every thread, before its first access to global memory
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            int it = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < p.total; w += gridDim.x) {
                const Work wk = decode(p, w);
                for (int kb = wk.kb0; kb < wk.kb1; kb++, it++) {
                    const int st = it % kStages;
                    if (it >= kStages && !mbar_wait(&sm.empty[st], ((it / kStages) - 1) & 1, ctx, SITE_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&sm.full[st], kATileBytes + kBTileBytes);
                    // K-major: map {contraction, rows}, one box {32, 128}.  MN-major: map {rows, contraction},
                    // four boxes {32, 32}: blocks of 32 rows, each [32 contraction steps x 128 bytes].
                    if (kAMN) {
                        if (p.a_one) {
                            tma_load_4d(sm.a[st], &map_a, &sm.full[st], 0, kb * kBK, wk.m0 / 32, 0);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                tma_load_4d(sm.a[st] + i * 4096, &map_a, &sm.full[st], wk.m0 + 32 * i, kb * kBK, 0, 0);
                        }
                    } else {
                        tma_load_4d(sm.a[st], &map_a, &sm.full[st], kb * kBK, wk.m0, 0, 0);
                    }
                    if (kBMN) {
                        if (p.b_one) {
                            tma_load_4d(sm.b[st], &map_b, &sm.full[st], 0, kb * kBK, wk.n0 / 32, 0);
                        } else {
#pragma unroll
                            for (int i = 0; i < kBN / 32; i++)
                                tma_load_4d(sm.b[st] + i * 4096, &map_b, &sm.full[st], wk.n0 + 32 * i, kb * kBK, 0, 0);
                        }
                    } else {
                        tma_load_4d(sm.b[st], &map_b, &sm.full[st], kb * kBK, wk.n0, 0, 0);  // the B map's box is kBN rows
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        constexpr uint32_t idesc = idesc_tf32(kBM, kBN, kAMN ? 1 : 0, kBMN ? 1 : 0);
        const uint32_t leader = elect_leader();
        int it = 0, j = 0;
        bool ok = true;
        for (int w = blockIdx.x; ok && w < p.total; w += gridDim.x, j++) {
            const Work wk = decode(p, w);
            const int acc = j & 1;
            if (j >= 2 && !mbar_wait_warp(&sm.acc_empty[acc], ((j >> 1) - 1) & 1, ctx, SITE_ACC_EMPTY)) break;
            tc_fence_after_sync();
            const uint32_t d = tmem + (uint32_t)acc * kBN;
            for (int kb = wk.kb0; kb < wk.kb1; kb++, it++) {
                const int st = it % kStages;
                if (!mbar_wait_warp(&sm.full[st], (it / kStages) & 1, ctx, SITE_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // MN-major tiles: 32-row blocks 4096 bytes apart, groups of 4 contraction steps 512 bytes apart
                const uint64_t ad = kAMN ? smem_desc_sw128_base32(smem_u32(sm.a[st]), 4096, 512)
                                         : smem_desc_sw128(smem_u32(sm.a[st]), 16, 1024);
                const uint64_t bd = kBMN ? smem_desc_sw128_base32(smem_u32(sm.b[st]), 4096, 512)
                                         : smem_desc_sw128(smem_u32(sm.b[st]), 16, 1024);
#pragma unroll
                for (int k = 0; k < kBK / 8; k++)
                    mma_tf32_lead(leader, d, desc_advance(ad, k * (kAMN ? 1024 : 32)),
                                  desc_advance(bd, k * (kBMN ? 1024 : 32)), idesc, (kb > wk.kb0 || k > 0) ? 1u : 0u);
                tc_commit_lead(leader, &sm.empty[st]);
            }
            if (ok) tc_commit_lead(leader, &sm.acc_full[acc]);
        }
    } else if (warp >= 4) {
        // ------------------------------ epilogue ------------------------------
        // Two warps per tensor-memory lane quarter: each thread owns one row and 32 of the 64 columns
        // of a chunk.  Warp 3 drives the copy engine.
        const int quarter = warp & 3;
        const int half = (warp - 4) >> 2;
        const int row = (quarter << 5) | lane;
        const uint32_t lane_addr = (uint32_t)(quarter << 5) << 16;
        int j = 0, chunk_count = 0;
        int sub = 0;  // stagings handed to the copy engine so far (one per chunk, two with the planes)
        bool ok = true;
        for (int w = blockIdx.x; ok && w < p.total; w += gridDim.x, j++) {
            const Work wk = decode(p, w);
            const int acc = j & 1;
            if (!mbar_wait_warp(&sm.acc_full[acc], (j >> 1) & 1, ctx, SITE_ACC_FULL)) break;
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < kBN / 64; c++, chunk_count++) {
                const int col0 = wk.n0 + 64 * c + 32 * half;  // first of this thread's 32 columns
                uint32_t r2[2][16];
#define R(i) r2[(i) >> 4][(i) & 15]
#pragma unroll
                for (int q = 0; q < 2; q++)
                    tmem_ld16(tmem + lane_addr + (uint32_t)acc * kBN + 64 * c + 32 * half + 16 * q, r2[q]);
                tmem_wait_ld();
                if (c == kBN / 64 - 1) {  // the accumulator has been read out: the tensor cores may reuse it
                    tc_fence_before_sync();
                    mbar_arrive(&sm.acc_empty[acc]);
                }
                if (kEpi == 0 && bias != nullptr) {
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        if (kDirect) {  // N need not be a multiple of 4: element-wise and guarded
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                if (col0 + 4 * q + e < p.N)
                                    R(4 * q + e) = __float_as_uint(__uint_as_float(R(4 * q + e)) + __ldg(bias + col0 + 4 * q + e));
                        } else if (col0 + 4 * q < p.N) {  // N is a multiple of 4
                            const float4 bv = __ldg(reinterpret_cast<const float4 *>(bias + col0) + q);
                            R(4 * q) = __float_as_uint(__uint_as_float(R(4 * q)) + bv.x);
                            R(4 * q + 1) = __float_as_uint(__uint_as_float(R(4 * q + 1)) + bv.y);
                            R(4 * q + 2) = __float_as_uint(__uint_as_float(R(4 * q + 2)) + bv.z);
                            R(4 * q + 3) = __float_as_uint(__uint_as_float(R(4 * q + 3)) + bv.w);
                        }
                    }
                }
                uint32_t hp[16], lp[16];  // packed bf16 pairs of the two planes
                if (kEpi == 0 && kPlanes) {
#pragma unroll
                    for (int e = 0; e < 16; e++) {
                        const float f0 = __uint_as_float(R(2 * e)), f1 = __uint_as_float(R(2 * e + 1));
                        const __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
                        const __nv_bfloat162 ll = __floats2bfloat162_rn(f0 - __low2float(hh), f1 - __high2float(hh));
                        hp[e] = *reinterpret_cast<const uint32_t *>(&hh);
                        lp[e] = *reinterpret_cast<const uint32_t *>(&ll);
                    }
                }
                if (kOut1) {
                    // one staging buffer: the two column halves of the chunk go through it one after the other
#pragma unroll 1
                    for (int hsel = 0; hsel < 2; hsel++) {
                        if (sub >= 1 && !mbar_wait_warp(&sm.out_free, (sub - 1) & 1, ctx, SITE_OUT_FREE)) {
                            ok = false;
                            break;
                        }
                        if (half == hsel) {
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                uint8_t *dst = sm.out[0] + row * 128 + ((q ^ (row & 7)) << 4);
                                *reinterpret_cast<uint4 *>(dst) = make_uint4(R(4 * q), R(4 * q + 1), R(4 * q + 2), R(4 * q + 3));
                            }
                        }
                        fence_proxy_async_smem();
                        mbar_arrive(&sm.out_ready);
                        sub++;
                    }
                    if (!ok) break;
                    continue;
                }
                // the copy engine must have read the previous staging out of the two buffers
                if (sub >= 1 && !mbar_wait_warp(&sm.out_free, (sub - 1) & 1, ctx, SITE_OUT_FREE)) {
                    ok = false;
                    break;
                }
#pragma unroll
                for (int q = 0; q < 8; q++) {  // fp32: this half's box of 32 columns, 8 chunks of 16 bytes per row
                    uint8_t *dst = sm.out[kOut1 ? 0 : half] + row * 128 + ((q ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(R(4 * q), R(4 * q + 1), R(4 * q + 2), R(4 * q + 3));
                }
#undef R
                if (kDirect) {
                    // every row of the staged chunk is written by one warp instruction: 32 consecutive floats
                    mbar_arrive(&sm.out_ready);
                    if (!mbar_wait_warp(&sm.out_ready, sub & 1, ctx, SITE_OUT_READY)) {
                        ok = false;
                        break;
                    }
                    const int et = threadIdx.x - 128;  // 0..255
                    const int cbase = wk.n0 + 64 * c;
#pragma unroll 4
                    for (int k = 0; k < (128 * 64) / kEpiThreads; k++) {
                        const int e = et + kEpiThreads * k;
                        const int rr = e >> 6, cc = e & 63;
                        const float v = *reinterpret_cast<const float *>(sm.out[kOut1 ? 0 : (cc >> 5)] + rr * 128 +
                                                                         ((((cc & 31) >> 2) ^ (rr & 7)) << 4) + ((cc & 3) << 2));
                        if (wk.m0 + rr < p.M && cbase + cc < p.N) c_direct[(size_t)(wk.m0 + rr) * p.N + cbase + cc] = v;
                    }
                    mbar_arrive(&sm.out_free);
                    sub++;
                } else {
                    fence_proxy_async_smem();
                    mbar_arrive(&sm.out_ready);
                    sub++;
                    if (kEpi == 0 && kPlanes) {
                        // second round: once the fp32 tiles have been read, the same buffers take the planes
                        if (!mbar_wait_warp(&sm.out_free, (sub - 1) & 1, ctx, SITE_OUT_FREE)) {
                            ok = false;
                            break;
                        }
#pragma unroll
                        for (int q = 0; q < 4; q++) {  // this half's 32 columns = 4 chunks of 8 bf16 values
                            const int off = row * 128 + (((4 * half + q) ^ (row & 7)) << 4);
                            *reinterpret_cast<uint4 *>(sm.out[0] + off) =
                                make_uint4(hp[4 * q], hp[4 * q + 1], hp[4 * q + 2], hp[4 * q + 3]);
                            *reinterpret_cast<uint4 *>(sm.out[kOut1 ? 0 : 1] + off) =
                                make_uint4(lp[4 * q], lp[4 * q + 1], lp[4 * q + 2], lp[4 * q + 3]);
                        }
                        fence_proxy_async_smem();
                        mbar_arrive(&sm.out_ready);
                        sub++;
                    }
                }
            }
        }
    } else if (warp == 3 && !kDirect) {
        // ------------------------------ output copies ------------------------------
        if (lane == 0) {
            int sub = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < p.total; w += gridDim.x) {
                const Work wk = decode(p, w);
                for (int c = 0; c < kBN / 64; c++) {
                    const int col0 = wk.n0 + 64 * c;
                    if (!mbar_wait(&sm.out_ready, sub & 1, ctx, SITE_OUT_READY)) {
                        ok = false;
                        break;
                    }
                    sub++;
                    if (kOut1) {  // one buffer, two rounds of 32 columns
                        if (kEpi == 0) tma_store_3d(sm.out[0], &map_c, col0, wk.m0, 0);
                        else tma_reduce_add_3d(sm.out[0], &map_c, col0, wk.m0, 0);
                        bulk_commit();
                        bulk_wait_read_all();
                        mbar_arrive(&sm.out_free);
                        if (!mbar_wait(&sm.out_ready, sub & 1, ctx, SITE_OUT_READY)) {
                            ok = false;
                            break;
                        }
                        sub++;
                        if (kEpi == 0) tma_store_3d(sm.out[0], &map_c, col0 + 32, wk.m0, 0);
                        else tma_reduce_add_3d(sm.out[0], &map_c, col0 + 32, wk.m0, 0);
                    } else if (kEpi == 0) {
                        tma_store_3d(sm.out[0], &map_c, col0, wk.m0, 0);
                        tma_store_3d(sm.out[kOut1 ? 0 : 1], &map_c, col0 + 32, wk.m0, 0);
                        if (kPlanes) {  // second round through the same buffers: hi plane, lo plane
                            bulk_commit();
                            bulk_wait_read_all();
                            mbar_arrive(&sm.out_free);
                            if (!mbar_wait(&sm.out_ready, sub & 1, ctx, SITE_OUT_READY)) {
                                ok = false;
                                break;
                            }
                            sub++;
                            tma_store_3d(sm.out[0], &map_planes, col0, wk.m0, 0);
                            tma_store_3d(sm.out[kOut1 ? 0 : 1], &map_planes, col0, wk.m0, 1);
                        }
                    } else {
                        tma_reduce_add_3d(sm.out[0], &map_c, col0, wk.m0, 0);
                        tma_reduce_add_3d(sm.out[kOut1 ? 0 : 1], &map_c, col0 + 32, wk.m0, 0);
                    }
                    bulk_commit();
                    bulk_wait_read_all();
                    mbar_arrive(&sm.out_free);
                }
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    if (sm.abort_flag) __nanosleep(50000);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// db[n] += sum_m dy[m, n].  A block covers 128 columns (one float4 per lane) and every 8th row of its
// share of the rows; four loads are in flight per thread.  N is a multiple of 4.
__global__ void __launch_bounds__(256) bias_grad_kernel(const float *__restrict__ dy, float *__restrict__ db, int M, int N,
                                                        int pitch) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    __shared__ float4 part[8][32];
    const int lane = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int col = blockIdx.x * 128 + 4 * lane;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < N) {
        const int step = gridDim.y * 8;
        int m = blockIdx.y * 8 + rl;
        for (; m + 3 * step < M; m += 4 * step) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldcs(reinterpret_cast<const float4 *>(dy + (size_t)(m + u * step) * pitch + col));
#pragma unroll
            for (int u = 0; u < 4; u++) acc.x += v[u].x, acc.y += v[u].y, acc.z += v[u].z, acc.w += v[u].w;
        }
        for (; m < M; m += step) {
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(dy + (size_t)m * pitch + col));
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
    }
    part[rl][lane] = acc;
    __syncthreads();
    if (rl == 0 && col < N) {
        float4 t = part[0][lane];
#pragma unroll
        for (int i = 1; i < 8; i++) t.x += part[i][lane].x, t.y += part[i][lane].y, t.z += part[i][lane].z, t.w += part[i][lane].w;
        atomicAdd(db + col, t.x);
        if (col + 1 < N) atomicAdd(db + col + 1, t.y);
        if (col + 2 < N) atomicAdd(db + col + 2, t.z);
        if (col + 3 < N) atomicAdd(db + col + 3, t.w);
    }
}

// dst[M, Np] = src[M, N] with zero columns N..Np-1: a copy of dy whose rows start on 16-byte boundaries, for
// outputs of layers whose feature count is not a multiple of 4 (the vocabulary projection).
__global__ void __launch_bounds__(256) pad_rows_kernel(float *__restrict__ dst, const float *__restrict__ src, int M, int N,
                                                       int Np) {
    tc05::pdl_launch_dependents();
    tc05::pdl_wait();
    // One block per row at a time.  The source row starts `o` floats past a 16-byte boundary (src itself is
    // 16-byte aligned): every thread loads the two aligned 16-byte words around its four values and picks them
    // out, so that loads and stores are all 16 bytes wide (the neighbour thread's copy of a word comes from L1).
    // Four such pairs are in flight per thread.  Words that reach past the end of src are read value by value.
    const size_t total = (size_t)M * N;
    const int nv = Np >> 2;
    auto load_word = [&](size_t at) -> float4 {
        if (at + 3 < total) return __ldg(reinterpret_cast<const float4 *>(src + at));
        float4 t;
        t.x = at < total ? src[at] : 0.f;
        t.y = at + 1 < total ? src[at + 1] : 0.f;
        t.z = at + 2 < total ? src[at + 2] : 0.f;
        t.w = at + 3 < total ? src[at + 3] : 0.f;
        return t;
    };
    constexpr int kU = 4;
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        const size_t start = (size_t)m * N;
        const int o = (int)(start & 3);
        const size_t base = start - o;  // multiple of 4
        float4 *out = reinterpret_cast<float4 *>(dst + (size_t)m * Np);
        for (int j0 = threadIdx.x; j0 < nv; j0 += 256 * kU) {
            float4 a[kU], b[kU];
#pragma unroll
            for (int u = 0; u < kU; u++) {
                const int j4 = j0 + 256 * u;
                a[u] = b[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j4 < nv) {
                    a[u] = load_word(base + 4 * (size_t)j4);
                    if (o != 0) b[u] = load_word(base + 4 * (size_t)(j4 + 1));
                }
            }
#pragma unroll
            for (int u = 0; u < kU; u++) {
                const int j4 = j0 + 256 * u;
                if (j4 >= nv) continue;
                const float v[8] = {a[u].x, a[u].y, a[u].z, a[u].w, b[u].x, b[u].y, b[u].z, b[u].w};
                float r[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float pick = o == 0 ? v[e] : (o == 1 ? v[e + 1] : (o == 2 ? v[e + 2] : v[e + 3]));
                    r[e] = 4 * j4 + e < N ? pick : 0.f;
                }
                __stcs(out + j4, make_float4(r[0], r[1], r[2], r[3]));
            }
        }
    }
}

// ---- host side ----

// Operand read K-major: matrix [rows, kc] row-major (kc contiguous = contraction); boxes of 32 x box_rows.
int map_k_major(CUtensorMap *map, const float *base, int rows, int kc, int box_rows) {
    const cuuint64_t dims[4] = {(cuuint64_t)kc, (cuuint64_t)rows, 1, 1};
    const cuuint64_t strides[3] = {(cuuint64_t)kc * 4, (cuuint64_t)kc * 4 * (cuuint64_t)rows, (cuuint64_t)kc * 4 * (cuuint64_t)rows};
    const cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
    return attn::encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box);
}
// Operand read MN-major, whole tile in one copy: the matrix [kc, rows] seen as {32 values, kc, rows / 32 blocks}
// with the block index as the slowest box dimension, box {32, 32, nblocks}: shared memory receives
// [block][contraction step][32 values], the layout the descriptor expects.  rows % 32 == 0.
int map_mn_major_blocks(CUtensorMap *map, const float *base, int kc, int rows, int nblocks) {
    const cuuint64_t dims[4] = {32, (cuuint64_t)kc, (cuuint64_t)(rows / 32), 1};
    const cuuint64_t strides[3] = {(cuuint64_t)rows * 4, 128, (cuuint64_t)rows * 4 * (cuuint64_t)kc};
    const cuuint32_t box[4] = {32, 32, (cuuint32_t)nblocks, 1};
    return attn::encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}
// Operand read MN-major: matrix [kc, rows] row-major (rows contiguous, kc = contraction), boxes of 32 x 32.
int map_mn_major(CUtensorMap *map, const float *base, int kc, int rows) {
    const cuuint64_t dims[4] = {(cuuint64_t)rows, (cuuint64_t)kc, 1, 1};
    const cuuint64_t strides[3] = {(cuuint64_t)rows * 4, (cuuint64_t)rows * 4 * (cuuint64_t)kc, (cuuint64_t)rows * 4 * (cuuint64_t)kc};
    const cuuint32_t box[4] = {32, 32, 1, 1};
    // 32-bit operands read MN-major need the 128-byte swizzle with 32-byte atoms (rows of 128 bytes, the
    // 32-byte quarter of a row XORed with the row index modulo 4)
    return attn::encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}
int map_out_f32(CUtensorMap *map, const float *base, int rows, int cols) {
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)cols * 4 * (cuuint64_t)rows};
    const cuuint32_t box[3] = {32, 128, 1};
    return attn::encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box);
}
int map_out_planes(CUtensorMap *map, const void *base, int rows, int cols) {
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 2};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)attn::plane_bytes((size_t)rows * cols)};
    const cuuint32_t box[3] = {64, 128, 1};
    return attn::encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box);
}

Problem make_problem(int M, int N, int K, int bn, int splits) {
    Problem p;
    p.M = M, p.N = N, p.K = K, p.bn = bn;
    p.a_one = p.b_one = 0;
    p.m_fast = 0;
    p.tiles_m = (M + kBM - 1) / kBM;
    p.tiles_n = (N + bn - 1) / bn;
    p.kb_total = (K + kBK - 1) / kBK;
    if (splits < 1) splits = 1;
    if (splits > p.kb_total) splits = p.kb_total;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;  // every split is non-empty
    p.total = p.tiles_m * p.tiles_n * p.splits;
    return p;
}

int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

// Tile width for a [M, N] result: the candidate with the fewest (rounds over the SMs) x (tile width),
// with a fixed charge per tile that makes narrow tiles pay for their higher operand traffic per flop.
int pick_bn(int M, int N, int splits, int sms) {
    const int cand[3] = {256, 192, 128};
    int best = 128;
    long long best_cost = -1;
    for (int i = 0; i < 3; i++) {
        const int bn = cand[i];
        if (bn > 128 && N < bn) continue;
        const long long tiles = (long long)((M + kBM - 1) / kBM) * ((N + bn - 1) / bn) * splits;
        const long long rounds = (tiles + sms - 1) / sms;
        const long long cost = rounds * (bn + 192);  // measured: a 192-wide tile costs ~0.9 of a 256-wide one
        if (best_cost < 0 || cost < best_cost) best = bn, best_cost = cost;
    }
    return best;
}

template <bool kAMN, bool kBMN, int kEpi, int kBN, int kStages, bool kPlanes, bool kDirect = false>
int launch_one(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const CUtensorMap &mp,
               const float *bias, const Problem &p, int *status, cudaStream_t s, float *c_direct = nullptr) {
    using Smem = SmemT<kBN, kStages, kPlanes>;
    static_assert(sizeof(Smem) <= 227 * 1024, "shared memory of the Linear kernel");
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    auto kernel = linear_gemm_kernel<kAMN, kBMN, kEpi, kBN, kStages, kPlanes, kDirect>;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
        if (e != cudaSuccess) return (int)e;
        attr_done[dev] = true;
    }
    const int sms = sm_count();
    const int grid = p.total < sms ? p.total : sms;
    return (int)attn::launch_after_previous(kernel, dim3(grid), dim3(kThreads), sizeof(Smem), s, ma, mb, mc, mp, bias, c_direct, p,
                                            status);
}

// Pipeline depth by what fits in 227 KiB next to the output staging tile.
template <bool kAMN, bool kBMN, int kEpi>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const CUtensorMap &mp, const float *bias,
           bool planes, const Problem &p, int *status, cudaStream_t s) {
    if (p.bn == 256) {
        if (planes) return launch_one<kAMN, kBMN, kEpi, 256, 4, true>(ma, mb, mc, mp, bias, p, status, s);
        return launch_one<kAMN, kBMN, kEpi, 256, 4, false>(ma, mb, mc, mp, bias, p, status, s);
    }
    if (p.bn == 192) {
        if (planes) return launch_one<kAMN, kBMN, kEpi, 192, 4, true>(ma, mb, mc, mp, bias, p, status, s);
        return launch_one<kAMN, kBMN, kEpi, 192, 5, false>(ma, mb, mc, mp, bias, p, status, s);
    }
    if (planes) return launch_one<kAMN, kBMN, kEpi, 128, 6, true>(ma, mb, mc, mp, bias, p, status, s);
    return launch_one<kAMN, kBMN, kEpi, 128, 6, false>(ma, mb, mc, mp, bias, p, status, s);
}

// C[M, N] = A[M, K] . B[N, K]^T: true when B (the weight) is too large to stay in L2 while every tile row of
// C passes over it and A is the smaller operand; the work items then run down the rows of C, so that B is read
// from HBM once and A (small) is what stays in L2.  (The vocabulary projection: B is 154 MB, A 25 MB.)
int stream_rows_of_c(int M, int N, int K) {
    const size_t a_bytes = (size_t)M * K * 4, b_bytes = (size_t)N * K * 4;
    return b_bytes > ((size_t)48 << 20) && b_bytes > a_bytes ? 1 : 0;
}

// Number of pieces the contraction of a [M, N] result is cut into when it is very long and the tiles do not
// fill the SMs evenly (dx of the vocabulary projection: 192 tiles on 148 SMs, 1571 steps each).  Each piece
// pays a fixed charge for its epilogue; 1 = no split.
int pick_splits(int tiles, int kb_total, int sms) {
    if (kb_total < 512) return 1;
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 8; s++) {
        const long long rounds = ((long long)tiles * s + sms - 1) / sms;
        const long long cost = rounds * ((kb_total + s - 1) / s + 24);
        if (best_cost < 0 || cost < best_cost) best = s, best_cost = cost;
    }
    return best;
}

// The same choice for dW, whose contraction (the rows of dy) is always cut: up to 32 pieces.
int pick_splits_dw(int tiles, int kb_total, int sms, int overhead) {
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 32 && s <= kb_total; s++) {
        const long long rounds = ((long long)tiles * s + sms - 1) / sms;
        const long long cost = rounds * ((kb_total + s - 1) / s + overhead);
        if (best_cost < 0 || cost < best_cost) best = s, best_cost = cost;
    }
    return best;
}

bool aligned16(const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

}  // namespace
}  // namespace lin

extern "C" {

int linear_sm100_forward(const float *x, const float *w, const float *bias, float *y, void *planes, int M, int N, int K,
                         void *stream) {
    using namespace lin;
    if (!x || !w || !y) return ATTN_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (long long)M * N > 0x7fffffffLL || (long long)M * K > 0x7fffffffLL) return ATTN_ERR_SHAPE;
    const bool direct = N % 4 != 0;  // y's rows are not 16-byte aligned: no copy engine for the output
    if (K % 4 != 0 || (planes && N % 8 != 0)) return ATTN_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(w) || (!direct && (!aligned16(y) || (bias && !aligned16(bias)))) ||
        (planes && !aligned16(planes)))
        return ATTN_ERR_ALIGN;
    int *status = nullptr;
    int rc = attn::device_status_word(&status);
    if (rc != ATTN_OK) return rc;
    CUtensorMap ma, mb, mc, mp;
    const int bn = direct ? 256 : pick_bn(M, N, 1, sm_count());
    if ((rc = map_k_major(&ma, x, M, K, 128)) != 0) return rc;
    if ((rc = map_k_major(&mb, w, N, K, bn)) != 0) return rc;
    if (direct) {
        Problem pd = make_problem(M, N, K, 256, 1);
        pd.m_fast = stream_rows_of_c(M, N, K);
        return launch_one<false, false, 0, 256, 4, false, true>(ma, mb, ma, ma, bias, pd, status,
                                                                static_cast<cudaStream_t>(stream), y);
    }
    if ((rc = map_out_f32(&mc, y, M, N)) != 0) return rc;
    mp = mc;
    if (planes && (rc = map_out_planes(&mp, planes, M, N)) != 0) return rc;
    Problem p = make_problem(M, N, K, bn, 1);
    p.m_fast = stream_rows_of_c(M, N, K);
    return launch<false, false, 0>(ma, mb, mc, mp, bias, planes != nullptr, p, status, static_cast<cudaStream_t>(stream));
}

size_t linear_sm100_backward_scratch_bytes(int M, int N, int K) {
    (void)K;
    if (M <= 0 || N <= 0 || N % 32 == 0) return 0;
    const size_t np = ((size_t)N + 31) / 32 * 32;
    return (size_t)M * np * sizeof(float);
}

int linear_sm100_backward(const float *dy, const float *x, const float *w, float *dx, float *dw, float *db, void *scratch,
                          int M, int N, int K, void *stream) {
    using namespace lin;
    if (!dy || !w || (!dx && !dw) || (dw && !x)) return ATTN_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (long long)M * N > 0x7fffffffLL || (long long)M * K > 0x7fffffffLL) return ATTN_ERR_SHAPE;
    if (K % 32 != 0) return ATTN_ERR_UNSUPPORTED;
    const bool padded = N % 32 != 0;  // dy's rows cannot be tiles of the copy engine as they are: work on a padded copy
    const int np = (N + 31) / 32 * 32;
    if ((long long)M * np > 0x7fffffffLL) return ATTN_ERR_SHAPE;
    if (padded && !scratch) return ATTN_ERR_NULL;
    // dy itself must start on a 16-byte boundary in both cases: the padding kernel reads it in 16-byte words
    if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx) || !aligned16(dw) ||
        (!padded && !aligned16(db)) || !aligned16(scratch))
        return ATTN_ERR_ALIGN;
    int *status = nullptr;
    int rc = attn::device_status_word(&status);
    if (rc != ATTN_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int sms = sm_count();
    const float *g = dy;  // [M, np] from here on
    if (padded) {
        rc = (int)attn::launch_after_previous(pad_rows_kernel, dim3(sms * 16), dim3(256), 0, s, static_cast<float *>(scratch), dy, M,
                                              N, np);
        if (rc != 0) return rc;
        g = static_cast<const float *>(scratch);
    }
    CUtensorMap ma, mb, mc;
    if (dx) {
        // dx[M,K] = dy[M,N] . w[N,K]: contraction over N (rows of w past N read as zeros)
        if ((rc = map_k_major(&ma, g, M, np, 128)) != 0) return rc;
        int bn_dx = pick_bn(M, K, 1, sms), splits_dx = 1;
        if (np / kBK >= 512) {  // very long contraction: tile width and number of pieces together
            const int cand[3] = {256, 192, 128};
            long long best_cost = -1;
            for (int i = 0; i < 3; i++) {
                if (cand[i] > 128 && K < cand[i]) continue;
                const int tiles = ((M + kBM - 1) / kBM) * ((K + cand[i] - 1) / cand[i]);
                const int sp = pick_splits(tiles, np / kBK, sms);
                const long long rounds = ((long long)tiles * sp + sms - 1) / sms;
                const long long cost = rounds * ((np / kBK + sp - 1) / sp + 24) * (cand[i] + 192);
                if (best_cost < 0 || cost < best_cost) best_cost = cost, bn_dx = cand[i], splits_dx = sp;
            }
        }
        Problem pdx = make_problem(M, K, np, bn_dx, splits_dx);
        pdx.b_one = map_mn_major_blocks(&mb, w, N, K, pdx.bn / 32) == 0;
        if (!pdx.b_one && (rc = map_mn_major(&mb, w, N, K)) != 0) return rc;
        if ((rc = map_out_f32(&mc, dx, M, K)) != 0) return rc;
        if (pdx.splits > 1) {
            // the pieces of the contraction add into dx with bulk reductions: start from zeros
            if ((rc = tensor_sm100_fill(dx, (size_t)M * K, 0.f, stream)) != 0) return rc;
            rc = launch<false, true, 1>(ma, mb, mc, mc, nullptr, false, pdx, status, s);
        } else {
            rc = launch<false, true, 0>(ma, mb, mc, mc, nullptr, false, pdx, status, s);
        }
        if (rc != 0) return rc;
    }
    if (dw) {
        // dw[N,K] += dy[M,N]^T . x[M,K]: contraction over M, split so that every SM has work (rows of the
        // result past N are dropped by the copy engine)
        const int bn = K % 256 == 0 ? 256 : (K % 192 == 0 ? 192 : 128);
        const int tiles = ((N + kBM - 1) / kBM) * ((K + bn - 1) / bn);
        // pieces of the contraction: whole rounds over the SMs cost (steps per piece + a fixed charge for the
        // piece's epilogue and reduction) each; e.g. QKV: 54 tiles, 256 steps -> 5 pieces in 2 rounds of 52 steps
        const int splits = pick_splits_dw(tiles, (M + kBK - 1) / kBK, sms, 8);
        Problem pdw = make_problem(N, K, M, bn, splits);
        pdw.a_one = map_mn_major_blocks(&ma, g, M, np, 4) == 0;
        if (!pdw.a_one && (rc = map_mn_major(&ma, g, M, np)) != 0) return rc;
        pdw.b_one = map_mn_major_blocks(&mb, x, M, K, bn / 32) == 0;
        if (!pdw.b_one && (rc = map_mn_major(&mb, x, M, K)) != 0) return rc;
        if ((rc = map_out_f32(&mc, dw, N, K)) != 0) return rc;
        rc = launch<true, true, 1>(ma, mb, mc, mc, nullptr, false, pdw, status, s);
        if (rc != 0) return rc;
    }
    if (db) {
        const int by = M >= 2048 ? 32 : (M + 63) / 64;  // rows per block column: at least 8 per row lane
        dim3 grid((unsigned)((N + 127) / 128), (unsigned)by);
        rc = (int)attn::launch_after_previous(bias_grad_kernel, grid, dim3(256), 0, s, g, db, M, N, np);
    }
    return rc;
}

}  // extern "C"
