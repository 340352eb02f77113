// Fused causal attention backward for sm_100a, head size 64.
//
// Replaces attention_backward_cuda_kernel of gpt.c (kernels/src/cuda/Attention.cu:235-324): the
// dO unpermute, the four batched SGEMMs, the in-place softmax backward over [B,H,T,T] and the
// permute-accumulate become one kernel that recomputes the probabilities from the saved
// log-sum-exp and never writes a T x T matrix.
//
// One CTA owns one (batch, head) and one tile of 128 keys (K_j, V_j stay in shared memory) and
// walks the query tiles i = j .. last.  Everything is computed transposed so that the key index
// is the tensor-memory lane:
//     S^T  = K_j Q_i^T            dP^T = V_j dO_i^T                 (B = Q / dO half, K-major)
//     P^T  = exp2(S^T * c - lse_i)        dS^T = P^T * (dP^T - delta_i)      (one thread per key)
//     dV_j += P^T dO_i            dK_j += dS^T Q_i                  (A from tensor memory)
//     dQ_i  = dS K_j                                                (A = dS^T tile in shared
//                                                                    memory read MN-major)
// dK_j and dV_j accumulate in tensor memory over the whole loop and leave once through bulk
// tensor stores; dQ_i is staged as an fp32 tile in shared memory and added into the (zeroed) dq
// third of the output by bulk tensor reductions, since other key tiles contribute to the same
// rows.  Every product is hi*hi + hi*lo + lo*hi on bf16 pairs.
//
// Each query tile is processed as two halves of 64 queries (A, B) with their own barriers, so the
// tensor cores and the compute warps overlap: while the compute warps turn S^T/dP^T of half B
// into P^T/dS^T, the tensor cores already run dV/dK of half A, the previous tile's dQ and the
// next tile's scores.
//
// Warp roles (640 threads):
//   warp 0      TMA producer: K, V once; Q/dO half tiles through a ring of three slots
//   warp 1      issues the score MMAs (S^T, dP^T), in order
//   warp 2      allocates tensor memory; stages the row statistics (-lse, -delta) of every query
//               tile; drives the output copies (dQ reductions, final dK / dV stores)
//   warp 3      issues the gradient MMAs (dV, dK per half; dQ per tile), whichever is ready first
//   warps 4-19  compute.  A compute warp's quarter (warp % 4) selects the 32 tensor-memory lanes
//               it may touch (keys for S^T / dP^T / dK / dV, queries for dQ); its column group
//               (0..3) selects 16 of the 64 query columns of a half and 16 of the 64 columns of
//               dQ / dK / dV.
// Two issuing warps on two schedulers, each electing its issuing lane once: a single issuing warp
// competes with four busy compute warps for its scheduler's issue slots and feeds the tensor pipe
// at well under its rate.  Dependencies between the two (a score task overwrites the columns a
// gradient task read) go through completion barriers, not through issue order.
//
// Tensor memory: S^T [0,128)  dP^T [128,256)  dV [256,320)  dK [320,384)  dQ [384,448)
// K hi [448,480)  V hi [480,512).  The hi planes of K and V are copied there once so that two of
// the three terms of S^T and dP^T take their A operand from tensor memory: an MMA with both
// operands in shared memory is limited by shared-memory bandwidth (48 instead of 32 cycles at
// N = 64).  P^T and dS^T overwrite S^T and dP^T in place: each run of 16 columns becomes 8 columns
// of packed bf16 hi parts followed by 8 columns of packed lo parts.
#include "attn_internal.h"
#include "tc05.cuh"

namespace attn {
namespace {

using namespace tc05;

constexpr int kTile = 128;
constexpr int kHalf = 64;
constexpr int kD = 64;
constexpr int kPlaneTile = kTile * kD * 2;  // 16 KiB: one bf16 plane of a 128-row tile
constexpr int kPlaneHalf = kHalf * kD * 2;  // 8 KiB
constexpr int kSlots = 3;                   // Q/dO half tiles in flight
constexpr int kThreads = 640;
constexpr int kGradWarp = 3;
constexpr int kComputeThreads = 512;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColST = 0, kColDPT = 128, kColDV = 256, kColDK = 320, kColDQ = 384, kColKH = 448, kColVH = 480;

struct __align__(1024) BwdSmem {
    uint8_t k[2][kPlaneTile];      // K_j   [plane]
    uint8_t v[2][kPlaneTile];      // V_j
    uint8_t in[kSlots][4][kPlaneHalf];  // ring of query half tiles: [slot][Q hi, Q lo, dO hi, dO lo][64 rows]
    // dS^T [plane][query half][128 keys x 64 queries].  Between two dQ products the first 32 KiB
    // also stage the finished fp32 dQ tile on its way out: [32-column half][128 queries x 128 bytes].
    uint8_t ds[2][2][kPlaneTile];
    float lse2[2][kTile];          // -log-sum-exp of the query tile in log2 units, double buffered
    float delta[2][kTile];         // -rowsum(dO * O)
    uint64_t kv_full;
    uint64_t in_full[kSlots], in_empty[kSlots];
    uint64_t st_full[2], pds_full[2];                       // [half]
    uint64_t ds_full;                                       // dS^T of both halves is in shared memory
    uint64_t dq_full[2];                                    // [iteration parity]
    uint64_t out_full, out_free;                            // staged dQ tile: written / read by the copy engine
    uint64_t kv_out_full;                                   // staged dK / dV tiles written
    uint64_t stats_full[2], stats_free[2], kv_tmem;  // [statistics buffer]
    uint32_t tmem_base;
    int abort_flag;
};

enum Site : int {
    SITE_IN_EMPTY = 101, SITE_IN_FULL, SITE_KV_FULL, SITE_ST_FULL, SITE_DQ_FULL_FREE, SITE_DQ_FULL_LAST, SITE_ROW_BAR,
    SITE_MMA_IDLE, SITE_STATS_FREE, SITE_KV_TMEM, SITE_OUT_FULL, SITE_OUT_FREE, SITE_SMEM_ALIGN
};

// Optional cycle trace of CTA 0 (debug builds with -DATTN_TRACE only).
#ifdef ATTN_TRACE
__device__ long long g_bwd_trace[2 * 16 * 8];
#define BWD_TRACE(cond, role, it, k)                                                              \
    do {                                                                                          \
        if (blockIdx.x == 0 && (cond)) g_bwd_trace[((role) * 16 + (it)) * 8 + (k)] = clock64();  \
    } while (0)
// life time of every 48th CTA in ns: rows 8..15 of role 1 are reused: [cta / 48][0..2]
__device__ long long g_bwd_life[16 * 4];
__device__ long long g_bwd_epi[8];
#define BWD_EPI(k) do { if (blockIdx.x == 0 && threadIdx.x == 128) g_bwd_epi[k] = (long long)global_timer_ns(); } while (0)
#define BWD_EPI2(k) do { if (blockIdx.x == 0) g_bwd_epi[k] = (long long)global_timer_ns(); } while (0)
#define BWD_LIFE(k)                                                                          \
    do {                                                                                     \
        if (threadIdx.x == 128 && blockIdx.x % 48 == 0)                                      \
            g_bwd_life[(blockIdx.x / 48) * 4 + (k)] = (long long)global_timer_ns();          \
    } while (0)
#else
#define BWD_EPI(k) do {} while (0)
#define BWD_EPI2(k) do {} while (0)
#define BWD_LIFE(k) \
    do {            \
    } while (0)
#define BWD_TRACE(cond, role, it, k) \
    do {                             \
    } while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// P^T and dS^T of 16 query columns starting at local query index q_base (thread = key `row`).
// Reads S^T / dP^T from tensor memory, writes the packed hi/lo pairs back in place and leaves
// the dS^T pairs in dh/dl for the shared-memory copy.
__device__ __forceinline__ void compute_run(const BwdSmem &sm, uint32_t t_st, uint32_t t_dpt, int lb, int q_base, int row,
                                            bool diag, float2 sc2, uint32_t (&dh)[8], uint32_t (&dl)[8]) {
    uint32_t sv[16], dp[16];
    tmem_ld16(t_st, sv);
    tmem_ld16(t_dpt, dp);
    tmem_wait_ld();
    uint32_t ph[8], pl[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const int q0 = q_base + 2 * e;
        const float2 nl = *reinterpret_cast<const float2 *>(&sm.lse2[lb][q0]);   // -lse * log2(e)
        const float2 nd = *reinterpret_cast<const float2 *>(&sm.delta[lb][q0]);  // -delta
        const float2 x = fma2(make_float2(__uint_as_float(sv[2 * e]), __uint_as_float(sv[2 * e + 1])), sc2, nl);
        float2 p = make_float2(ex2(x.x), ex2(x.y));
        if (diag) {  // causal: a query sees a key only when query >= key
            if (q0 < row) p.x = 0.f;
            if (q0 + 1 < row) p.y = 0.f;
        }
        const float2 d = mul2(p, add2(make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])), nd));
        split_bf16x2_packed(p, ph[e], pl[e]);
        split_bf16x2_packed(d, dh[e], dl[e]);
    }
    tmem_st8(t_st, ph);
    tmem_st8(t_st + 8, pl);
    tmem_st8(t_dpt, dh);
    tmem_st8(t_dpt + 8, dl);
}

// dS^T row `row`, 16 queries of column group cq, into the 128-byte-swizzled MN-major tile of one
// query half: 16-byte chunk index (2 * cq + g) ^ (row % 8).
__device__ __forceinline__ void store_ds(uint8_t *tile_h, uint8_t *tile_l, int row, int cq, const uint32_t (&dh)[8],
                                         const uint32_t (&dl)[8]) {
#pragma unroll
    for (int g2 = 0; g2 < 2; g2++) {
        const int chunk = ((2 * cq + g2) ^ (row & 7)) * 16;
        *reinterpret_cast<uint4 *>(tile_h + row * 128 + chunk) =
            make_uint4(dh[4 * g2], dh[4 * g2 + 1], dh[4 * g2 + 2], dh[4 * g2 + 3]);
        *reinterpret_cast<uint4 *>(tile_l + row * 128 + chunk) =
            make_uint4(dl[4 * g2], dl[4 * g2 + 1], dl[4 * g2 + 2], dl[4 * g2 + 3]);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_dx, const float *__restrict__ lse, const float *__restrict__ delta, float *__restrict__ dqkv, int B, int T,
                int H, float scale, float scale_log2, int *status) {
    // The structure fills the whole 227 KiB, so there is no room to round the base up: the
    // swizzled tiles need 1024-byte alignment and the kernel refuses to run without it.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    BwdSmem &sm = *reinterpret_cast<BwdSmem *>(smem_raw);
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_TIMEOUT_BASE + SITE_SMEM_ALIGN);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = B * H;
    const int nt = (T + kTile - 1) / kTile;
    const int jt = (int)(blockIdx.x / BH);  // key tile; tile 0 has the most work and goes first
    const int bh = (int)(blockIdx.x % BH);
    const int b = bh / H, h = bh % H;
    const int C = H * kD;
    const int niter = nt - jt;  // query tiles jt .. nt-1

    WaitCtx ctx{&sm.abort_flag, status};
    pdl_launch_dependents();
    BWD_LIFE(0);

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.kv_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm.st_full[i], 1);
            mbar_init(&sm.pds_full[i], kComputeThreads);
            mbar_init(&sm.dq_full[i], 1);
        }
        for (int i = 0; i < kSlots; i++) {
            mbar_init(&sm.in_full[i], 1);
            mbar_init(&sm.in_empty[i], 1);
        }
        mbar_init(&sm.ds_full, kComputeThreads);
        mbar_init(&sm.stats_full[0], 32);
        mbar_init(&sm.stats_full[1], 32);
        mbar_init(&sm.stats_free[0], kComputeThreads / 32);
        mbar_init(&sm.stats_free[1], kComputeThreads / 32);
        mbar_init(&sm.kv_tmem, kComputeThreads);
        mbar_init(&sm.out_full, kComputeThreads);
        mbar_init(&sm.out_free, 1);
        mbar_init(&sm.kv_out_full, kComputeThreads);
        fence_barrier_init();
        // This thread is also the TMA producer: K, V and the first Q/dO half tiles are requested
        // right away, while the other warps are still setting up (but not before the kernel that
        // wrote them has completed).
        pdl_wait();
        fence_proxy_async_smem();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_do);
        const int xq = h * kD, xk = C + h * kD, xv = 2 * C + h * kD;
        mbar_expect_tx(&sm.kv_full, 4 * kPlaneTile);
        for (int hf = 0; hf < 2; hf++) {
            for (int pl = 0; pl < 2; pl++) {
                tma_load_4d(sm.k[pl] + hf * kPlaneHalf, &map_x, &sm.kv_full, xk, jt * kTile + hf * kHalf, b, pl);
                tma_load_4d(sm.v[pl] + hf * kPlaneHalf, &map_x, &sm.kv_full, xv, jt * kTile + hf * kHalf, b, pl);
            }
        }
        for (int t = 0; t < kSlots && t < 2 * niter; t++) {
            const int y = (jt + (t >> 1)) * kTile + (t & 1) * kHalf;
            mbar_expect_tx(&sm.in_full[t], 4 * kPlaneHalf);
            tma_load_4d(sm.in[t][0], &map_x, &sm.in_full[t], xq, y, b, 0);
            tma_load_4d(sm.in[t][1], &map_x, &sm.in_full[t], xq, y, b, 1);
            tma_load_4d(sm.in[t][2], &map_do, &sm.in_full[t], h * kD, y, b, 0);
            tma_load_4d(sm.in[t][3], &map_do, &sm.in_full[t], h * kD, y, b, 1);
        }
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
        // ------------------------------ TMA producer (boxes of 64 rows) ------------------------------
        if (lane == 0) {
            const int xq = h * kD;
            // Half tile t = 2n + half goes to slot t % 3 (the first three were requested during
            // set-up); a slot is free again once the dV / dK products that read it have completed.
            for (int t = kSlots, slot = 0, use = 1; t < 2 * niter; t++) {
                if (!mbar_wait(&sm.in_empty[slot], (use - 1) & 1, ctx, SITE_IN_EMPTY)) break;
                const int y = (jt + (t >> 1)) * kTile + (t & 1) * kHalf;
                mbar_expect_tx(&sm.in_full[slot], 4 * kPlaneHalf);
                tma_load_4d(sm.in[slot][0], &map_x, &sm.in_full[slot], xq, y, b, 0);
                tma_load_4d(sm.in[slot][1], &map_x, &sm.in_full[slot], xq, y, b, 1);
                tma_load_4d(sm.in[slot][2], &map_do, &sm.in_full[slot], h * kD, y, b, 0);
                tma_load_4d(sm.in[slot][3], &map_do, &sm.in_full[slot], h * kD, y, b, 1);
                if (++slot == kSlots) { slot = 0; use++; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer: S^T, dP^T ------------------------------
        constexpr uint32_t idesc_st = idesc_bf16_f32(kTile, kHalf, 0, 0);  // S^T, dP^T of one half (N = 64)
        // K-major views (rows of 64 head-dim values)
        const uint64_t k_km[2] = {smem_desc_sw128(smem_u32(sm.k[0]), 16, 1024), smem_desc_sw128(smem_u32(sm.k[1]), 16, 1024)};
        const uint64_t v_km[2] = {smem_desc_sw128(smem_u32(sm.v[0]), 16, 1024), smem_desc_sw128(smem_u32(sm.v[1]), 16, 1024)};
        // Q/dO ring: descriptors of slot 0, plane 0; slot s, plane p lies (4 s + p) * 8 KiB further
        const uint64_t in_km = smem_desc_sw128(smem_u32(sm.in[0][0]), 16, 1024);

        // Score tasks t = 2n + half, in order: S^T and dP^T of one half of a query tile.  Task t
        // overwrites the columns task t-2 produced, so the dV / dK products that consumed those
        // (gradient task t-2, issued by another warp) must have completed.
        bool ok = mbar_wait_warp(&sm.kv_tmem, 0, ctx, SITE_KV_TMEM);
        tc_fence_after_sync();
        const uint32_t leader = elect_leader();  // the one lane that issues every MMA and commit of this warp
        int s_slot = 0, s_use = 0, e_slot = 0, e_use = 0;
        for (int t = 0; ok && t < 2 * niter; t++) {
            const int hf = t & 1;
            [[maybe_unused]] const int n = t >> 1;  // only the trace build reads it
            if (t >= 2) {
                ok = mbar_wait_warp(&sm.in_empty[e_slot], e_use & 1, ctx, SITE_IN_EMPTY);
                if (++e_slot == kSlots) { e_slot = 0; e_use++; }
            }
            ok = ok && mbar_wait_warp(&sm.in_full[s_slot], s_use & 1, ctx, SITE_IN_FULL);
            if (!ok) break;
            const uint64_t q_km = desc_advance(in_km, s_slot * 4 * kPlaneHalf);
            const uint64_t g_km = desc_advance(q_km, 2 * kPlaneHalf);
            tc_fence_after_sync();
            BWD_TRACE(lane == 0, 0, n, 0 + 4 * hf);
            uint32_t acc = 0;
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                for (int kk = 0; kk < kD / 16; kk++) {
                    if (term < 2)
                        mma_ts_lead(leader, tmem + kColST + hf * kHalf, tmem + kColKH + 8 * kk,
                                     desc_advance(q_km, bb * kPlaneHalf + kk * 32), idesc_st, acc);
                    else
                        mma_ss_lead(leader, tmem + kColST + hf * kHalf, desc_advance(k_km[a], kk * 32),
                                     desc_advance(q_km, bb * kPlaneHalf + kk * 32), idesc_st, acc);
                    acc = 1;
                }
            }
            acc = 0;
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                for (int kk = 0; kk < kD / 16; kk++) {
                    if (term < 2)
                        mma_ts_lead(leader, tmem + kColDPT + hf * kHalf, tmem + kColVH + 8 * kk,
                                     desc_advance(g_km, bb * kPlaneHalf + kk * 32), idesc_st, acc);
                    else
                        mma_ss_lead(leader, tmem + kColDPT + hf * kHalf, desc_advance(v_km[a], kk * 32),
                                     desc_advance(g_km, bb * kPlaneHalf + kk * 32), idesc_st, acc);
                    acc = 1;
                }
            }
            tc_commit_lead(leader, &sm.st_full[hf]);
            BWD_TRACE(lane == 0, 0, n, 1 + 4 * hf);
            if (++s_slot == kSlots) { s_slot = 0; s_use++; }
        }
    } else if (warp == 2) {
        // ------------------------------ row statistics and output copies ------------------------------
        // Two small jobs polled by one warp.  (1) -lse * log2(e) and -delta of every query tile,
        // double buffered in shared memory; each buffer has its own full / free barriers, so this
        // warp can never be two phases ahead of a reader of the same barrier.  (2) Staged dQ tiles
        // are added into dqkv (several key tiles contribute to one query tile), the final dK / dV
        // tiles are plain stores; rows past the end of the sequence are dropped by the copy engine.
        if (lane == 0) tma_prefetch_desc(&map_dx);
        const int xq = h * kD, xk = C + h * kD, xv = 2 * C + h * kD;
        int m = 0, o = 0;
        bool kv_stored = false, ok = true;
        uint64_t idle_since = 0;
        uint32_t idle_polls = 0;
        while (ok && !(kv_stored && o == niter)) {
            bool progressed = false;
            if (m < niter) {
                const int buf = m & 1;
                if (m < 2 || __all_sync(0xffffffffu, mbar_test_wait(&sm.stats_free[buf], ((m >> 1) - 1) & 1))) {
#pragma unroll
                    for (int k = 0; k < kTile / 32; k++) {
                        const int r = lane + 32 * k, t = (jt + m) * kTile + r;
                        sm.lse2[buf][r] = t < T ? -lse[(size_t)bh * T + t] * 1.4426950408889634f : 0.f;
                        sm.delta[buf][r] = t < T ? -delta[(size_t)bh * T + t] : 0.f;
                    }
                    mbar_arrive(&sm.stats_full[buf]);
                    m++;
                    progressed = true;
                }
            }
            if (o < niter) {
                if (__all_sync(0xffffffffu, mbar_test_wait(&sm.out_full, o & 1))) {
                    if (lane == 0) {
                        tma_reduce_add_3d(sm.ds[0][0], &map_dx, xq, (jt + o) * kTile, b);
                        tma_reduce_add_3d(sm.ds[0][1], &map_dx, xq + 32, (jt + o) * kTile, b);
                        bulk_commit();
                        if (o == niter - 1) BWD_EPI2(1);
                        bulk_wait_read_all();
                        if (o == niter - 1) BWD_EPI2(5);
                        mbar_arrive(&sm.out_free);
                    }
                    __syncwarp();
                    o++;
                    progressed = true;
                }
            }
            if (!kv_stored && __all_sync(0xffffffffu, mbar_test_wait(&sm.kv_out_full, 0))) {
                if (lane == 0) {
                    tma_store_3d(sm.in[0][0], &map_dx, xk, jt * kTile, b);
                    tma_store_3d(sm.in[0][2], &map_dx, xk + 32, jt * kTile, b);
                    tma_store_3d(sm.in[1][0], &map_dx, xv, jt * kTile, b);
                    tma_store_3d(sm.in[1][2], &map_dx, xv + 32, jt * kTile, b);
                    bulk_commit();
                    BWD_EPI2(6);
                }
                kv_stored = true;
                progressed = true;
            }
            if (progressed) {
                idle_polls = 0;
            } else if ((++idle_polls & 255u) == 0u) {  // bounded: give up when nothing became ready for a second
                const uint64_t now = global_timer_ns();
                if (idle_polls == 256u) idle_since = now;
                const bool give_up = (now - idle_since > TC05_WAIT_LIMIT_NS) || sm.abort_flag;
                if (__any_sync(0xffffffffu, give_up)) {
                    if (lane == 0 && !sm.abort_flag) {
                        sm.abort_flag = 1;
                        if (status) atomicCAS(status, 0, ST_TIMEOUT_BASE + SITE_OUT_FULL);
                    }
                    ok = false;
                }
            }
        }
        // Shared memory must stay alive until the copies have read it; the writes themselves
        // complete on their own before the grid does.
        if (lane == 0) bulk_wait_read_all();
        if (lane == 0) BWD_EPI2(7);
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------ compute group ------------------------------
        const int quarter = warp & 3;
        const int cq = (warp - 4) >> 2;           // column group: 16 query columns of each half
        const int row = (quarter << 5) | lane;    // key inside the tile == TMEM lane; query row for dQ
        const uint32_t lane_addr = (uint32_t)(quarter << 5) << 16;
        const uint32_t t_st = tmem + lane_addr + kColST + 16 * cq;
        const uint32_t t_dpt = tmem + lane_addr + kColDPT + 16 * cq;
        bool ok = true;

        // One row (16 of its 64 columns) of an fp32 output tile into the staging layout the copy
        // engine expects: two 32-column halves, 128-byte rows, 16-byte chunks swizzled by row % 8.
        auto stage_row = [&](uint8_t *tile, const uint32_t (&r)[16], float f) {
            uint8_t *base = tile + (cq >> 1) * kPlaneTile + row * 128;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int chunk = ((4 * (cq & 1) + e) ^ (row & 7)) * 16;
                *reinterpret_cast<float4 *>(base + chunk) =
                    make_float4(__uint_as_float(r[4 * e]) * f, __uint_as_float(r[4 * e + 1]) * f,
                                __uint_as_float(r[4 * e + 2]) * f, __uint_as_float(r[4 * e + 3]) * f);
            }
        };
        // dQ of iteration n (its barrier phase has been waited for): scale this thread's 16 columns
        // into the staging tile; warp 3 adds the tile into dqkv with one bulk reduction per half.
        auto flush_dq = [&](int n) -> bool {
            tc_fence_after_sync();
            uint32_t r[16];
            tmem_ld16(tmem + lane_addr + kColDQ + 16 * cq, r);
            tmem_wait_ld();
            stage_row(sm.ds[0][0], r, scale);
            fence_proxy_async_smem();
            mbar_arrive(&sm.out_full);
            return true;
        };

        // K hi and V hi, this thread's 16 head-dim values of key `row`, into tensor memory (packed
        // pairs, so 8 columns each); the rows in shared memory are 128-byte swizzled.
        if (!mbar_wait_warp(&sm.kv_full, 0, ctx, SITE_KV_FULL)) ok = false;
        if (ok) {
            uint32_t kh[8], vh[8];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int off = row * 128 + (((2 * cq + j) ^ (row & 7)) << 4);
                const uint4 a = *reinterpret_cast<const uint4 *>(sm.k[0] + off);
                const uint4 c = *reinterpret_cast<const uint4 *>(sm.v[0] + off);
                kh[4 * j] = a.x, kh[4 * j + 1] = a.y, kh[4 * j + 2] = a.z, kh[4 * j + 3] = a.w;
                vh[4 * j] = c.x, vh[4 * j + 1] = c.y, vh[4 * j + 2] = c.z, vh[4 * j + 3] = c.w;
            }
            tmem_st8(tmem + lane_addr + kColKH + 8 * cq, kh);
            tmem_st8(tmem + lane_addr + kColVH + 8 * cq, vh);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.kv_tmem);
        }
        BWD_LIFE(1);
        const float2 sc2 = make_float2(scale_log2, scale_log2);
        for (int n = 0; ok && n < niter; n++) {
            const bool diag = (n == 0);
            const int lb = n & 1;
            // row statistics of this query tile (warp 2 stages them up to two tiles ahead)
            if (!mbar_wait_warp(&sm.stats_full[lb], (n >> 1) & 1, ctx, SITE_ROW_BAR)) { ok = false; break; }

            uint32_t dh_a[8], dl_a[8], dh_b[8], dl_b[8];
            // half A: queries 0..63 of the tile
            BWD_TRACE(threadIdx.x == 128, 1, n, 0);
            if (!mbar_wait_warp(&sm.st_full[0], n & 1, ctx, SITE_ST_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            BWD_TRACE(threadIdx.x == 128, 1, n, 1);
            compute_run(sm, t_st, t_dpt, lb, 16 * cq, row, diag, sc2, dh_a, dl_a);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.pds_full[0]);  // dV / dK of half A may start; dS^T goes to shared memory below
            BWD_TRACE(threadIdx.x == 128, 1, n, 2);
            // While the tensor cores work on half B's scores: the previous tile's dQ (issued as soon as
            // its dS^T was stored) has finished by now; move it out.  The copy engine reads the staged
            // tile while half B is computed, then dS^T of this tile may overwrite it.
            if (n >= 1) {
                if (!mbar_wait_warp(&sm.dq_full[(n - 1) & 1], ((n - 1) >> 1) & 1, ctx, SITE_DQ_FULL_FREE)) {
                    ok = false;
                    break;
                }
                if (!flush_dq(n - 1)) { ok = false; break; }
            }
            BWD_TRACE(threadIdx.x == 128, 1, n, 7);
            // half B: queries 64..127
            if (!mbar_wait_warp(&sm.st_full[1], n & 1, ctx, SITE_ST_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            BWD_TRACE(threadIdx.x == 128, 1, n, 3);
            compute_run(sm, t_st + kHalf, t_dpt + kHalf, lb, kHalf + 16 * cq, row, diag, sc2, dh_b, dl_b);
            BWD_TRACE(threadIdx.x == 128, 1, n, 4);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.pds_full[1]);  // dV / dK of half B may start
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.stats_free[lb]);  // this warp has read the tile's statistics
            BWD_TRACE(threadIdx.x == 128, 1, n, 5);
            // the staged dQ tile of the previous iteration must have left shared memory
            if (n >= 1 && !mbar_wait_warp(&sm.out_free, (n - 1) & 1, ctx, SITE_OUT_FREE)) { ok = false; break; }
            store_ds(sm.ds[0][0], sm.ds[1][0], row, cq, dh_a, dl_a);
            store_ds(sm.ds[0][1], sm.ds[1][1], row, cq, dh_b, dl_b);
            fence_proxy_async_smem();
            mbar_arrive(&sm.ds_full);  // dQ may start
            BWD_TRACE(threadIdx.x == 128, 1, n, 6);
        }

        BWD_LIFE(2);
        BWD_EPI(0);
        // Epilogue.  Once the last dV / dK products have completed the Q/dO ring is dead: its space
        // stages the dK and dV tiles for the copy engine while the last dQ product still runs.
        const int last = 2 * niter - 1;
        if (ok && mbar_wait_warp(&sm.in_empty[last % kSlots], (last / kSlots) & 1, ctx, SITE_IN_EMPTY)) {
            tc_fence_after_sync();
            uint32_t rk[16], rv[16];
            tmem_ld16(tmem + lane_addr + kColDK + 16 * cq, rk);
            tmem_ld16(tmem + lane_addr + kColDV + 16 * cq, rv);
            tmem_wait_ld();
            BWD_EPI(3);
            stage_row(sm.in[0][0], rk, scale);
            stage_row(sm.in[1][0], rv, 1.f);
            fence_proxy_async_smem();
            mbar_arrive(&sm.kv_out_full);
            BWD_EPI(4);
            if (mbar_wait_warp(&sm.dq_full[(niter - 1) & 1], ((niter - 1) >> 1) & 1, ctx, SITE_DQ_FULL_LAST)) {
                flush_dq(niter - 1);
                BWD_EPI(2);
            }
        }
    } else if (warp == kGradWarp) {
        // ------------------------------ MMA issuer: dV, dK, dQ ------------------------------
        // Two task streams, each in order: gradient tasks g = 2n + half (dV, dK of one half, once the
        // compute warps have turned that half into P^T / dS^T) and one dQ task per query tile (once
        // dS^T is in shared memory).  Whichever is ready goes first, dQ before dV / dK: the compute
        // warps need its result, and its operand buffer, one tile later.
        constexpr uint32_t idesc_kv = idesc_bf16_f32(kTile, kD, 0, 1);  // dV, dK (A in TMEM)
        constexpr uint32_t idesc_dq = idesc_bf16_f32(kTile, kD, 1, 1);  // dQ (A, B MN-major)
        // MN-major views: the row index is the contraction index
        const uint64_t in_mn = smem_desc_sw128(smem_u32(sm.in[0][0]), 1024, 1024);
        const uint64_t k_mn[2] = {smem_desc_sw128(smem_u32(sm.k[0]), 1024, 1024), smem_desc_sw128(smem_u32(sm.k[1]), 1024, 1024)};
        const uint64_t ds_mn[2] = {smem_desc_sw128(smem_u32(sm.ds[0][0]), kPlaneTile, 1024),
                                   smem_desc_sw128(smem_u32(sm.ds[1][0]), kPlaneTile, 1024)};
        const int ntask = 2 * niter;
        int g_idx = 0, d_idx = 0, g_slot = 0;
        const uint32_t leader = elect_leader();
        bool ok = true;
        uint64_t idle_since = 0;
        uint32_t idle_polls = 0;
        while (ok && d_idx < niter) {
            bool progressed = false;
            if (2 * d_idx + 1 < g_idx) {
                // dQ_i = dS K_j over all 128 keys
                const int n = d_idx;
                if (__all_sync(0xffffffffu, mbar_test_wait(&sm.ds_full, n & 1))) {
                    tc_fence_after_sync();
                    BWD_TRACE(lane == 0, 1, 8 + (n & 7), 0);
                    const uint32_t d_q = tmem + kColDQ;
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                        for (int kk = 0; kk < kTile / 16; kk++) {
                            mma_ss_lead(leader, d_q, desc_advance(ds_mn[a], kk * 2048), desc_advance(k_mn[bb], kk * 2048),
                                        idesc_dq, (term > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    tc_commit_lead(leader, &sm.dq_full[n & 1]);
                    BWD_TRACE(lane == 0, 1, 8 + (n & 7), 1);
                    d_idx++;
                    progressed = true;
                }
            }
            if (g_idx < ntask) {
                const int n = g_idx >> 1, hf = g_idx & 1;
                if (__all_sync(0xffffffffu, mbar_test_wait(&sm.pds_full[hf], n & 1))) {
                    tc_fence_after_sync();
                    const uint64_t q_mn = desc_advance(in_mn, g_slot * 4 * kPlaneHalf);
                    const uint64_t g_mn = desc_advance(q_mn, 2 * kPlaneHalf);
                    BWD_TRACE(lane == 0, 0, n, 2 + 4 * hf);
                    // dV += P^T dO_i over this half's 64 queries (4 K-steps of 16)
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            const int kk = 4 * hf + k4;
                            mma_ts_lead(leader, tmem + kColDV, tmem + kColST + 16 * kk + 8 * a, desc_advance(g_mn, bb * kPlaneHalf + k4 * 2048),
                                         idesc_kv, (g_idx > 0 || term > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    // dK += dS^T Q_i
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            const int kk = 4 * hf + k4;
                            mma_ts_lead(leader, tmem + kColDK, tmem + kColDPT + 16 * kk + 8 * a, desc_advance(q_mn, bb * kPlaneHalf + k4 * 2048),
                                         idesc_kv, (g_idx > 0 || term > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    tc_commit_lead(leader, &sm.in_empty[g_slot]);
                    if (++g_slot == kSlots) g_slot = 0;
                    BWD_TRACE(lane == 0, 0, n, 3 + 4 * hf);
                    g_idx++;
                    progressed = true;
                }
            }
            if (progressed) {
                idle_polls = 0;
            } else if ((++idle_polls & 255u) == 0u) {  // bounded: give up when nothing became ready for a second
                const uint64_t now = global_timer_ns();
                if (idle_polls == 256u) idle_since = now;
                const bool give_up = (now - idle_since > TC05_WAIT_LIMIT_NS) || sm.abort_flag;
                if (__any_sync(0xffffffffu, give_up)) {
                    if (lane == 0 && !sm.abort_flag) {
                        sm.abort_flag = 1;
                        if (status) atomicCAS(status, 0, ST_TIMEOUT_BASE + SITE_MMA_IDLE);
                    }
                    ok = false;
                }
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    if (sm.abort_flag) __nanosleep(50000);
    BWD_EPI(4);
    tc_fence_before_sync();
    __syncthreads();
    BWD_LIFE(3);
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

#ifdef ATTN_TRACE
extern "C" int attn_bwd_trace_read(long long *dst) {
    return (int)cudaMemcpyFromSymbol(dst, g_bwd_trace, sizeof(g_bwd_trace));
}
extern "C" int attn_bwd_epi_read(long long *dst) {
    return (int)cudaMemcpyFromSymbol(dst, g_bwd_epi, sizeof(g_bwd_epi));
}
extern "C" int attn_bwd_life_read(long long *dst) {
    return (int)cudaMemcpyFromSymbol(dst, g_bwd_life, sizeof(g_bwd_life));
}
#endif

static size_t bwd_smem_bytes() { return sizeof(BwdSmem); }
static_assert(sizeof(BwdSmem) <= 227 * 1024, "backward kernel shared memory");

cudaError_t fast_bwd_set_attributes() {
    return cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem_bytes());
}

// map_x / map_do must have boxes of 64 rows (see the producer warp); map_dx covers dqkv as fp32
// {3C, T, B} with boxes of 32 columns x 128 rows, 128-byte swizzle.
cudaError_t launch_fast_backward(const CUtensorMap &map_x, const CUtensorMap &map_do, const CUtensorMap &map_dx, const float *lse,
                                 const float *delta, float *dqkv, int B, int T, int H, int *status, cudaStream_t s) {
    const int nt = (T + kTile - 1) / kTile;
    const unsigned grid = (unsigned)(nt * B * H);
    const float scale = 0.125f;  // 1/sqrt(64)
    return launch_after_previous(attn_bwd_kernel, dim3(grid), dim3(kThreads), bwd_smem_bytes(), s, map_x, map_do, map_dx, lse,
                                 delta, dqkv, B, T, H, scale, scale * 1.4426950408889634f, status);
}

}  // namespace attn
