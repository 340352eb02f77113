// Fused causal attention backward for sm_100a, head size 64.
//
// Replaces attention_backward_cuda_kernel of gpt.c (kernels/src/cuda/Attention.cu:235-324): the
// dO unpermute, the four batched SGEMMs, the in-place softmax backward over [B,H,T,T] and the
// permute-accumulate become one kernel that recomputes the probabilities from the saved
// log-sum-exp and never writes a T x T matrix.
//
// The kernel is persistent: one CTA per SM takes work items from a list.  A work item is one (batch,
// head) and one tile of 128 keys (K_j, V_j stay in shared memory) together with the query tiles
// i = j .. last.  Items are ordered heaviest first (key tile 0 sees every query tile); a CTA starts
// with the item of its own number, then its mirror image in the second round, and takes every
// further one from a counter in global memory, two to three items ahead of the one it works on, so
// an SM that runs slower than the others (the time of the same work differs by +-7 % between SMs)
// simply takes fewer of the small items at the end.  A fixed deal of the items left the slowest
// CTA 9 % behind the average.  Barriers, tensor memory and the Q/dO ring live for the whole launch;
// the K/V tiles of the next item are requested as soon as the last tensor-core instruction that
// reads the current ones has completed, so that set-up of item w+1 overlaps the drain of item w.
//
// The kernel is sensitive to the size of its code: five roles run their loops side by side on one
// SM, and with the time-out logic of every barrier wait inlined (88 KB of code instead of 74) every
// query tile took 7 % longer.  That logic is therefore one shared function (tc05.cuh), the items'
// numbers reach the roles through plain loads behind waits they perform anyway (ItemFeed), and the
// loops that issue the tensor-core instructions stay fully unrolled all the same: rolling up the
// three terms of a product, 6 KB less code, cost 22 % (the issuing thread then computes descriptors
// at run time).
//
// Everything is computed transposed so that the key index is the tensor-memory lane:
//     S^T  = K_j Q_i^T            dP^T = V_j dO_i^T                 (B = Q / dO half, K-major)
//     P^T  = exp2(S^T * c - lse_i)        dS^T = P^T * (dP^T - delta_i)      (one thread per key)
//     dV_j += P^T dO_i            dK_j += dS^T Q_i                  (A from tensor memory)
//     dQ_i  = dS K_j                                                (A = dS^T tile in shared
//                                                                    memory read MN-major)
// dK_j and dV_j accumulate in tensor memory over the whole item and leave once, staged in shared
// memory, through bulk tensor stores.  dQ_i leaves after every query tile: staged as fp32 in the
// dS^T buffer (the only 32 KiB that are ever free: the dQ product that read it has completed) and
// added into the (zeroed) dq third of the output by bulk tensor reductions, since other key tiles
// contribute to the same rows.  The copy engine takes ~2600 cycles to drain a tile of reductions
// and the next dS^T has to wait for that; the variants that were measured against this one all
// lost: staging half or all of the tile in the V hi plane (dead once it is in tensor memory),
// flushing after half B instead of after half A, and adding dQ from registers with red.global (one
// thread per row, or four lanes per row after a 16x256b tensor-memory load: the reductions back up
// into the compute warps, ~1900 cycles per tile).  Every product is hi*hi + hi*lo + lo*hi on bf16
// pairs.
//
// Each query tile is processed as two halves of 64 queries (A, B) with their own barriers, so the
// tensor cores and the compute warps overlap: while the compute warps turn S^T/dP^T of half B
// into P^T/dS^T, the tensor cores already run dV/dK of half A, the previous tile's dQ and the
// next tile's scores.
//
// Warp roles (640 threads):
//   warp 0      TMA producer: K, V of every item; Q/dO half tiles through a ring of three slots that
//               runs on across items
//   warp 1      issues the score MMAs (S^T, dP^T), in order
//   warp 2      allocates tensor memory; stages the row statistics (-lse, -delta) of every query
//               tile, two tiles ahead; drives the output copies (dQ reductions, dK / dV stores)
//   warp 3      issues the gradient MMAs in the order they become ready: dV, dK of half A, of
//               half B, then dQ of the tile
//   warps 4-19  compute.  A compute warp's quarter (warp % 4) selects the 32 tensor-memory lanes
//               it may touch (keys for S^T / dP^T / dK / dV, queries for dQ); its column group
//               (0..3) selects 16 of the 64 query columns of a half and 16 of the 64 columns of
//               dQ / dK / dV.
// Two issuing warps on two schedulers, each electing its issuing lane once: a single issuing warp
// competes with four busy compute warps for its scheduler's issue slots and feeds the tensor pipe
// at well under its rate.  Dependencies between the two (a score task overwrites the columns a
// gradient task read) go through completion barriers, not through issue order.  Every role blocks
// on the one barrier its next task needs (the order in which tasks become ready is fixed), so idle
// roles sleep in mbarrier.try_wait instead of polling.
//
// Tensor memory: S^T [0,128)  dP^T [128,256)  dV [256,320)  dK [320,384)  dQ [384,448)
// K hi [448,480)  V hi [480,512).  The hi planes of K and V are copied there once per item so that
// two of the three terms of S^T and dP^T take their A operand from tensor memory: an MMA with both
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
constexpr int kQueue = 4;  // a slot is rewritten when every role has long read it
constexpr int kMoreBit = 1 << 30;
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
    // one completion per work item
    uint64_t kv_full;     // K_j, V_j have landed in shared memory
    uint64_t kv_tmem;     // their hi planes have been copied to tensor memory
    uint64_t v_free;      // the item's last dP^T product has completed: V_j may be overwritten
    uint64_t k_free;      // the item's last dQ product has completed: K_j may be overwritten
    uint64_t grads_done;  // the item's last dV / dK product has completed
    uint64_t kv_out_full; // the item's dK / dV tiles are staged in two slots of the (then dead) Q/dO ring
    uint64_t stage_free;  // ... and the copy engine has read them
    // one completion per query tile: its dQ tile is staged / the copy engine has read it.  (Every waiter
    // sees every phase of the barriers it waits on: a parity wait cannot tell "the phase before mine is
    // still open" from "mine has completed".)
    uint64_t out_full, out_free;
    // one completion per half tile (ring) or per query tile
    uint64_t in_full[kSlots], in_empty[kSlots];
    uint64_t st_full[2], pds_full[2];  // [half]
    uint64_t ds_full;                  // dS^T of both halves is in shared memory
    uint64_t dq_full[2];               // [tile parity]
    uint64_t stats_full[2], stats_free[2];  // [statistics buffer]
    // The CTA's items in the order it takes them (ItemFeed).  q_raw[k % kQueue]: number of item k, or a
    // number past the end of the list; q_item[k % kQueue]: the same with kMoreBit set when item k + 1
    // exists, posted only for items that exist, one completion of q_full per post.
    uint64_t q_full[kQueue];
    int q_item[kQueue];
    int q_raw[kQueue];
    uint32_t tmem_base;
    int abort_flag;
};

enum Site : int {
    SITE_IN_EMPTY = 101, SITE_IN_FULL, SITE_KV_FULL, SITE_ST_FULL, SITE_DQ_FULL_FREE, SITE_DQ_FULL_LAST, SITE_ROW_BAR,
    SITE_PDS_FULL, SITE_STATS_FREE, SITE_KV_TMEM, SITE_DS_FULL, SITE_GRADS_DONE, SITE_SMEM_ALIGN, SITE_V_FREE, SITE_K_FREE,
    SITE_KV_OUT_FULL, SITE_STAGE_FREE, SITE_TMEM_BASE, SITE_OUT_FULL, SITE_OUT_FREE, SITE_QUEUE
};

// Item p of the list (0 = heaviest) is key tile p / BH of (batch, head) p % BH.
struct Work {
    int jt, bh, niter;
};
__device__ __forceinline__ Work decode_item(int p, int BH, int nt) {
    Work w;
    w.jt = p / BH;
    w.bh = p - w.jt * BH;
    w.niter = nt - w.jt;  // query tiles jt .. nt-1
    return w;
}

// How a role learns the CTA's items.  Item 0 is the CTA's own number and item 1 its mirror image in the
// second round (as in a snake deal), so the first entry needs no communication; entry k >= 1 is read from
// BwdSmem::q_item with a plain load once the role has passed the first barrier wait of item k that it
// performs anyway (the entry was posted more than an item earlier, and the poster has completed barriers
// the role has waited for since).  Keeping a barrier wait with its time-out out of the roles' item loops
// matters: with one in, the compiler's code for the compute warps ran 7 % slower.
struct ItemFeed {
    int p;      // number of the current item
    bool more;  // another item follows
    __device__ ItemFeed(int nitems) : p((int)blockIdx.x), more(2 * (int)gridDim.x - 1 - (int)blockIdx.x < nitems) {}
    // entry k (k >= 1); the caller has made sure it has been posted
    __device__ __forceinline__ void read(const BwdSmem &sm, uint32_t k) {
        const int e = *reinterpret_cast<const volatile int *>(&sm.q_item[k % kQueue]);
        p = e & (kMoreBit - 1);
        more = (e & kMoreBit) != 0;
    }
};

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
                const __grid_constant__ CUtensorMap map_dx, const float *__restrict__ lse, const float *__restrict__ delta,
                float *__restrict__ dqkv, int B, int T, int H, float scale, float scale_log2, int *sched, int *status) {
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
    const int C = H * kD;

    WaitCtx ctx{&sm.abort_flag, status};
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.kv_full, 1);
        mbar_init(&sm.kv_tmem, kComputeThreads);
        mbar_init(&sm.v_free, 1);
        mbar_init(&sm.k_free, 1);
        mbar_init(&sm.grads_done, 1);
        mbar_init(&sm.kv_out_full, kComputeThreads);
        mbar_init(&sm.stage_free, 1);
        mbar_init(&sm.out_full, kComputeThreads);
        mbar_init(&sm.out_free, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm.st_full[i], 1);
            mbar_init(&sm.pds_full[i], kComputeThreads);
            mbar_init(&sm.dq_full[i], 1);
            mbar_init(&sm.stats_full[i], 32);
            mbar_init(&sm.stats_free[i], kComputeThreads / 32);
        }
        for (int i = 0; i < kSlots; i++) {
            mbar_init(&sm.in_full[i], 1);
            mbar_init(&sm.in_empty[i], 1);
        }
        mbar_init(&sm.ds_full, kComputeThreads);
        for (int i = 0; i < kQueue; i++) mbar_init(&sm.q_full[i], 1);
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
    // The CTA owns all 512 columns of its SM's tensor memory, so the allocation starts at column 0, lane 0.
    // Using that as a constant keeps every tensor-memory address of the MMA issue loops out of the per-lane
    // registers (an address loaded from shared memory has to be moved to a uniform register before every
    // instruction that takes it); an allocation anywhere else is reported and the CTA does nothing.
    constexpr uint32_t tmem = 0;
    const bool tmem_ok = sm.tmem_base == tmem;
    ItemFeed feed(BH * nt);
    Work w;

    if (!tmem_ok) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_TIMEOUT_BASE + SITE_TMEM_BASE);
    } else if (warp == 0) {
        // ------------------------------ TMA producer (boxes of 64 rows) ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_x);
            tma_prefetch_desc(&map_do);
            // Half tile number g of the whole launch goes to ring slot g % 3; the slot is free again once
            // the dV / dK products that read its previous content have completed.
            uint32_t g = 0;
            bool ok = true;
            auto load_half = [&](const Work &it, int t) {
                const uint32_t slot = g % kSlots;
                if (g >= (uint32_t)kSlots && !mbar_wait(&sm.in_empty[slot], (g / kSlots - 1) & 1, ctx, SITE_IN_EMPTY)) {
                    ok = false;
                    return;
                }
                const int b = it.bh / H, h = it.bh % H;
                const int y = (it.jt + (t >> 1)) * kTile + (t & 1) * kHalf;
                mbar_expect_tx(&sm.in_full[slot], 4 * kPlaneHalf);
                tma_load_4d(sm.in[slot][0], &map_x, &sm.in_full[slot], h * kD, y, b, 0);
                tma_load_4d(sm.in[slot][1], &map_x, &sm.in_full[slot], h * kD, y, b, 1);
                tma_load_4d(sm.in[slot][2], &map_do, &sm.in_full[slot], h * kD, y, b, 0);
                tma_load_4d(sm.in[slot][3], &map_do, &sm.in_full[slot], h * kD, y, b, 1);
                g++;
            };
            auto load_kv = [&](const Work &it, uint8_t (*dst)[kPlaneTile], int x0) {
                const int b = it.bh / H;
                for (int hf = 0; hf < 2; hf++)
                    for (int pl = 0; pl < 2; pl++)
                        tma_load_4d(dst[pl] + hf * kPlaneHalf, &map_x, &sm.kv_full, x0, it.jt * kTile + hf * kHalf, b, pl);
            };
            Work nxt;
            bool has = true;
            w = decode_item(feed.p, BH, nt);
            mbar_expect_tx(&sm.kv_full, 4 * kPlaneTile);
            load_kv(w, sm.k, C + (w.bh % H) * kD);
            load_kv(w, sm.v, 2 * C + (w.bh % H) * kD);
            int pre = 0;  // half tiles of the current item already requested
            for (uint32_t item = 0; has && ok; item++) {
                for (int t = pre; ok && t < 2 * w.niter; t++) load_half(w, t);
                // the next item: its entry is the (item + 1)-th post, made while the CTA worked on the item
                // before this one
                const bool has_next = feed.more;
                if (has_next) {
                    if (!mbar_wait(&sm.q_full[(item + 1) % kQueue], ((item + 1) / kQueue) & 1, ctx, SITE_QUEUE)) break;
                    feed.read(sm, item + 1);
                    nxt = decode_item(feed.p, BH, nt);
                }
                pre = 0;
                if (has_next && ok) {
                    // The next item's tiles, each as soon as its destination is free: the first Q/dO half
                    // tile behind the third last one of this item, V behind the last dP^T product, K behind
                    // the last dQ product.
                    const int xh = (nxt.bh % H) * kD;
                    load_half(nxt, 0);
                    if (ok && !mbar_wait(&sm.v_free, item & 1, ctx, SITE_V_FREE)) ok = false;
                    if (ok) {
                        mbar_expect_tx(&sm.kv_full, 4 * kPlaneTile);
                        load_kv(nxt, sm.v, 2 * C + xh);
                    }
                    if (ok && !mbar_wait(&sm.k_free, item & 1, ctx, SITE_K_FREE)) ok = false;
                    if (ok) load_kv(nxt, sm.k, C + xh);
                    // the other two ring slots stage this item's dK / dV tiles on their way out
                    if (ok && !mbar_wait(&sm.stage_free, item & 1, ctx, SITE_STAGE_FREE)) ok = false;
                    pre = 1;
                }
                w = nxt;
                has = has_next;
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
        const uint32_t leader = elect_leader();  // the one lane that issues every MMA and commit of this warp

        // Score tasks in order: S^T and dP^T of one half of a query tile.  Task g (numbered over the
        // whole launch) overwrites the columns task g-2 produced, so the dV / dK products that consumed
        // those (gradient task g-2, issued by another warp) must have completed.
        uint32_t g = 0;
        bool ok = true;
        for (uint32_t item = 0; ok; item++) {
            ok = mbar_wait_warp(&sm.kv_tmem, item & 1, ctx, SITE_KV_TMEM);
            if (!ok) break;
            if (item > 0) feed.read(sm, item);
            w = decode_item(feed.p, BH, nt);
            for (int t = 0; ok && t < 2 * w.niter; t++, g++) {
                const int hf = t & 1;
                const uint32_t slot = g % kSlots;
                if (g >= 2) ok = mbar_wait_warp(&sm.in_empty[(g - 2) % kSlots], ((g - 2) / kSlots) & 1, ctx, SITE_IN_EMPTY);
                ok = ok && mbar_wait_warp(&sm.in_full[slot], (g / kSlots) & 1, ctx, SITE_IN_FULL);
                if (!ok) break;
                const uint64_t q_km = desc_advance(in_km, slot * 4 * kPlaneHalf);
                const uint64_t g_km = desc_advance(q_km, 2 * kPlaneHalf);
                tc_fence_after_sync();
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
                if (t == 2 * w.niter - 1) tc_commit_lead(leader, &sm.v_free);
            }
            if (!feed.more) break;
        }
    } else if (warp == 2) {
        // ------------------------------ row statistics and output copies ------------------------------
        // Two small jobs, taken in the fixed order in which the compute warps make them ready.
        // (1) -lse * log2(e) and -delta of every query tile, double buffered in shared memory: tile n
        // (numbered over the whole launch) goes to buffer n % 2 once every compute warp has released tile
        // n - 2; each buffer has its own full / free barriers, so this warp is never two phases ahead of a
        // reader.  (2) Staged dQ tiles are added into dqkv (several key tiles contribute to one query
        // tile), the dK / dV tiles of a finished item are plain stores; rows past the end of the sequence
        // are dropped by the copy engine.
        if (lane == 0) tma_prefetch_desc(&map_dx);
        // The query tiles of this CTA's items, in processing order.  This warp hands the items out (below)
        // and reads their numbers from q_raw, which it has written itself.
        const int nitems = BH * nt, G = (int)gridDim.x;
        struct TileCursor {
            Work w;
            int m;
            uint32_t item;
            bool valid, pending;
            __device__ TileCursor() : m(0), item(0), valid(true), pending(true) {}
            __device__ bool ready(const BwdSmem &sm, int BH, int nt) {  // all lanes, after a __syncwarp behind q_raw's writer
                if (pending) {
                    const int p = *reinterpret_cast<const volatile int *>(&sm.q_raw[item % kQueue]);
                    valid = p < BH * nt;
                    if (valid) w = decode_item(p, BH, nt);
                    pending = false;
                }
                return valid;
            }
            __device__ void advance() {
                if (++m >= w.niter) {
                    m = 0;
                    item++;
                    pending = true;
                }
            }
        };
        TileCursor cur, ahead;
        auto stage_stats = [&](const TileCursor &c, uint32_t n) {
            const int buf = n & 1;
#pragma unroll
            for (int k = 0; k < kTile / 32; k++) {
                const int r = lane + 32 * k, t = (c.w.jt + c.m) * kTile + r;
                sm.lse2[buf][r] = t < T ? -lse[(size_t)c.w.bh * T + t] * 1.4426950408889634f : 0.f;
                sm.delta[buf][r] = t < T ? -delta[(size_t)c.w.bh * T + t] : 0.f;
            }
            mbar_arrive(&sm.stats_full[buf]);
        };
        // Handing out the items.  The first two are fixed (ItemFeed); every further one comes from the
        // counter in global memory.  The number of item k + 3 is asked for when this warp begins the last query
        // tile of item k and used at the end of that tile's round, when the answer (a microsecond or two) has
        // long arrived: it goes to q_raw for this warp's own look-ahead of two query tiles, which therefore
        // never waits for a number, and it completes the entry of item k + 2, which tells the other roles
        // whether an item k + 3 follows.  The small items at the end of the list are thus still handed out
        // two or three at a time.  (The producer warp is the wrong place to ask: the request held up its
        // tile requests by over a thousand cycles.)
        auto ask = [&](int last_known) -> uint32_t {  // lane 0 holds the answer
            uint32_t ticket = 0;
            if (last_known < nitems && lane == 0)
                asm volatile("atom.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(sched) : "memory");
            return ticket;
        };
        auto answer = [&](int last_known, uint32_t ticket) -> int {
            return last_known < nitems ? 2 * G + (int)__shfl_sync(0xffffffffu, ticket, 0) : nitems;
        };
        // item `k` gets its number `p` in q_raw; the entry of item k - 1 (number `p_before`) is complete with it
        auto hand_out = [&](uint32_t k, int p, int p_before) {
            if (lane == 0) {
                sm.q_raw[k % kQueue] = p;
                if (p_before < nitems) {
                    sm.q_item[(k - 1) % kQueue] = p_before | (p < nitems ? kMoreBit : 0);
                    mbar_arrive(&sm.q_full[(k - 1) % kQueue]);  // releases the store above
                }
            }
            __syncwarp();
        };
        int p_last = 2 * G - 1 - (int)blockIdx.x;  // number of the last item known (item 1)
        uint32_t known = 2;  // items whose numbers are known
        if (lane == 0) {
            sm.q_raw[0] = (int)blockIdx.x;
            sm.q_raw[1] = p_last;
            sm.q_item[0] = (int)blockIdx.x | (p_last < nitems ? kMoreBit : 0);
            mbar_arrive(&sm.q_full[0]);
        }
        __syncwarp();
        {
            const uint32_t ticket = ask(p_last);
            for (uint32_t n = 0; n < 2 && ahead.ready(sm, BH, nt); n++) {
                stage_stats(ahead, n);
                ahead.advance();
            }
            const int p = answer(p_last, ticket);
            hand_out(known++, p, p_last);
            p_last = p;
        }
        // the staged dQ tile of query tile `qt` -> dq third of dqkv
        auto reduce_dq = [&](const Work &it, int qt) {
            if (lane == 0) {
                const int b = it.bh / H, xq = (it.bh % H) * kD;
                tma_reduce_add_3d(sm.ds[0][0], &map_dx, xq, qt * kTile, b);
                tma_reduce_add_3d(sm.ds[0][1], &map_dx, xq + 32, qt * kTile, b);
                bulk_commit();
                bulk_wait_read_all();
                mbar_arrive(&sm.out_free);
            }
            __syncwarp();
        };
        bool ok = true;
        uint32_t item = 0;  // items finished
        for (uint32_t n = 0; ok && cur.ready(sm, BH, nt); n++) {
            const bool last_tile = cur.m == cur.w.niter - 1;
            uint32_t ticket = 0;
            if (last_tile) ticket = ask(p_last);
            if (cur.m >= 1) {  // dQ of the item's previous query tile (staged after half A of this one)
                if (!mbar_wait_warp(&sm.out_full, (n - 1) & 1, ctx, SITE_OUT_FULL)) break;
                reduce_dq(cur.w, cur.w.jt + cur.m - 1);
            }
            if (ahead.ready(sm, BH, nt)) {  // statistics two tiles ahead, into the buffer tile n releases
                if (!mbar_wait_warp(&sm.stats_free[n & 1], (n >> 1) & 1, ctx, SITE_STATS_FREE)) break;
                stage_stats(ahead, n + 2);
                ahead.advance();
            }
            if (cur.m == cur.w.niter - 1) {  // end of the item: dK and dV, then the last dQ
                if (!mbar_wait_warp(&sm.kv_out_full, item & 1, ctx, SITE_KV_OUT_FULL)) break;
                if (lane == 0) {
                    // the ring slots of the item's last two half tiles (numbers 2n and 2n + 1 of the launch)
                    const uint32_t s_k = (2 * n) % kSlots, s_v = (2 * n + 1) % kSlots;
                    const int b = cur.w.bh / H, xk = C + (cur.w.bh % H) * kD, xv = xk + C;
                    tma_store_3d(sm.in[s_k][0], &map_dx, xk, cur.w.jt * kTile, b);
                    tma_store_3d(sm.in[s_k][2], &map_dx, xk + 32, cur.w.jt * kTile, b);
                    tma_store_3d(sm.in[s_v][0], &map_dx, xv, cur.w.jt * kTile, b);
                    tma_store_3d(sm.in[s_v][2], &map_dx, xv + 32, cur.w.jt * kTile, b);
                    bulk_commit();
                    bulk_wait_read_all();
                    mbar_arrive(&sm.stage_free);
                }
                __syncwarp();
                if (!mbar_wait_warp(&sm.out_full, n & 1, ctx, SITE_OUT_FULL)) break;
                reduce_dq(cur.w, cur.w.jt + cur.m);
                item++;
            }
            if (last_tile) {
                const int p = answer(p_last, ticket);
                hand_out(known++, p, p_last);
                p_last = p;
            }
            cur.advance();
        }
        // Shared memory must stay alive until the copies have read it (they have: every group was waited
        // for above); the writes themselves complete on their own before the grid does.
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------ compute group ------------------------------
        const int quarter = warp & 3;
        const int cq = (warp - 4) >> 2;           // column group: 16 query columns of each half
        const int row = (quarter << 5) | lane;    // key inside the tile == TMEM lane; query row for dQ
        const uint32_t lane_addr = (uint32_t)(quarter << 5) << 16;
        const uint32_t t_st = tmem + lane_addr + kColST + 16 * cq;
        const uint32_t t_dpt = tmem + lane_addr + kColDPT + 16 * cq;
        const float2 sc2 = make_float2(scale_log2, scale_log2);
        bool ok = true;
        uint32_t n = 0;  // query tiles processed so far in this launch

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
        // dQ of the last query tile (its barrier phase has been waited for): scale this thread's 16 columns
        // into the staging tile; warp 2 adds the tile into dqkv with one bulk reduction per half.
        auto flush_dq = [&]() {
            tc_fence_after_sync();
            uint32_t r[16];
            tmem_ld16(tmem + lane_addr + kColDQ + 16 * cq, r);
            tmem_wait_ld();
            stage_row(sm.ds[0][0], r, scale);
            fence_proxy_async_smem();
            mbar_arrive(&sm.out_full);
        };

        for (uint32_t item = 0; ok; item++) {
            // K hi and V hi, this thread's 16 head-dim values of key `row`, into tensor memory (packed
            // pairs, so 8 columns each); the rows in shared memory are 128-byte swizzled.  The previous
            // item's last score products, the readers of these columns, completed before this thread left
            // that item's loop.
            if (!mbar_wait_warp(&sm.kv_full, item & 1, ctx, SITE_KV_FULL)) { ok = false; break; }
            if (item > 0) feed.read(sm, item);
            w = decode_item(feed.p, BH, nt);
            {
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
            for (int m = 0; ok && m < w.niter; m++, n++) {
                const bool diag = (m == 0);
                const int lb = n & 1;
                // row statistics of this query tile (warp 2 stages them up to two tiles ahead)
                if (!mbar_wait_warp(&sm.stats_full[lb], (n >> 1) & 1, ctx, SITE_ROW_BAR)) { ok = false; break; }

                uint32_t dh_a[8], dl_a[8], dh_b[8], dl_b[8];
                // half A: queries 0..63 of the tile
                if (!mbar_wait_warp(&sm.st_full[0], n & 1, ctx, SITE_ST_FULL)) { ok = false; break; }
                tc_fence_after_sync();
                compute_run(sm, t_st, t_dpt, lb, 16 * cq, row, diag, sc2, dh_a, dl_a);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.pds_full[0]);  // dV / dK of half A may start; dS^T goes to shared memory below
                // While the tensor cores work on half B's scores: the previous tile's dQ (issued as soon as
                // its dS^T was stored) has finished by now; move it out.  The copy engine reads the staged
                // tile while half B is computed, then dS^T of this tile may overwrite it.
                if (m >= 1) {
                    if (!mbar_wait_warp(&sm.dq_full[(n - 1) & 1], ((n - 1) >> 1) & 1, ctx, SITE_DQ_FULL_FREE)) {
                        ok = false;
                        break;
                    }
                    flush_dq();
                }
                // half B: queries 64..127
                if (!mbar_wait_warp(&sm.st_full[1], n & 1, ctx, SITE_ST_FULL)) { ok = false; break; }
                tc_fence_after_sync();
                compute_run(sm, t_st + kHalf, t_dpt + kHalf, lb, kHalf + 16 * cq, row, diag, sc2, dh_b, dl_b);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.pds_full[1]);  // dV / dK of half B may start
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.stats_free[lb]);  // this warp has read the tile's statistics
                // the staged dQ tile of the previous query tile (of this item or the one before) must have left
                // shared memory
                if (n >= 1 && !mbar_wait_warp(&sm.out_free, (n - 1) & 1, ctx, SITE_OUT_FREE)) { ok = false; break; }
                store_ds(sm.ds[0][0], sm.ds[1][0], row, cq, dh_a, dl_a);
                store_ds(sm.ds[0][1], sm.ds[1][1], row, cq, dh_b, dl_b);
                fence_proxy_async_smem();
                mbar_arrive(&sm.ds_full);  // dQ may start
            }
            if (!ok) break;

            // End of the item.  Once the last dV / dK products have completed the Q/dO ring is dead except
            // for the slot the producer refills first: the slots of the item's last two half tiles stage
            // the dK and dV tiles for the copy engine while the last dQ product still runs; then that dQ.
            if (!mbar_wait_warp(&sm.grads_done, item & 1, ctx, SITE_GRADS_DONE)) { ok = false; break; }
            tc_fence_after_sync();
            {
                uint32_t rk[16], rv[16];
                tmem_ld16(tmem + lane_addr + kColDK + 16 * cq, rk);
                tmem_ld16(tmem + lane_addr + kColDV + 16 * cq, rv);
                tmem_wait_ld();
                stage_row(sm.in[(2 * n - 2) % kSlots][0], rk, scale);
                stage_row(sm.in[(2 * n - 1) % kSlots][0], rv, 1.f);
                fence_proxy_async_smem();
                mbar_arrive(&sm.kv_out_full);
            }
            if (!mbar_wait_warp(&sm.dq_full[(n - 1) & 1], ((n - 1) >> 1) & 1, ctx, SITE_DQ_FULL_LAST)) { ok = false; break; }
            flush_dq();
            tc_fence_before_sync();  // the reads above are ordered before the next item's arrivals
            if (!feed.more) break;
        }
    } else if (warp == kGradWarp) {
        // ------------------------------ MMA issuer: dV, dK, dQ ------------------------------
        // Per query tile, in the order the operands become ready: dV, dK of half A, of half B (once the
        // compute warps have turned that half into P^T / dS^T), then dQ of the tile (once dS^T is in shared
        // memory).
        constexpr uint32_t idesc_kv = idesc_bf16_f32(kTile, kD, 0, 1);  // dV, dK (A in TMEM)
        constexpr uint32_t idesc_dq = idesc_bf16_f32(kTile, kD, 1, 1);  // dQ (A, B MN-major)
        // MN-major views: the row index is the contraction index
        const uint64_t in_mn = smem_desc_sw128(smem_u32(sm.in[0][0]), 1024, 1024);
        const uint64_t k_mn[2] = {smem_desc_sw128(smem_u32(sm.k[0]), 1024, 1024), smem_desc_sw128(smem_u32(sm.k[1]), 1024, 1024)};
        const uint64_t ds_mn[2] = {smem_desc_sw128(smem_u32(sm.ds[0][0]), kPlaneTile, 1024),
                                   smem_desc_sw128(smem_u32(sm.ds[1][0]), kPlaneTile, 1024)};
        const uint32_t leader = elect_leader();
        uint32_t g = 0, n = 0;  // half tiles / query tiles issued so far in this launch
        bool ok = true;
        for (uint32_t item = 0; ok; item++) {
            // the item's entry has been posted and read by the compute warps before they arrive here
            if (!mbar_wait_warp(&sm.kv_tmem, item & 1, ctx, SITE_KV_TMEM)) break;
            if (item > 0) feed.read(sm, item);
            w = decode_item(feed.p, BH, nt);
            for (int m = 0; ok && m < w.niter; m++, n++) {
                for (int hf = 0; hf < 2; hf++, g++) {
                    if (!mbar_wait_warp(&sm.pds_full[hf], n & 1, ctx, SITE_PDS_FULL)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t slot = g % kSlots;
                    const uint64_t q_mn = desc_advance(in_mn, slot * 4 * kPlaneHalf);
                    const uint64_t g_mn = desc_advance(q_mn, 2 * kPlaneHalf);
                    const bool first = (m == 0 && hf == 0);  // the item's accumulators start from zero
                    // dV += P^T dO_i over this half's 64 queries (4 K-steps of 16)
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            const int kk = 4 * hf + k4;
                            mma_ts_lead(leader, tmem + kColDV, tmem + kColST + 16 * kk + 8 * a,
                                        desc_advance(g_mn, bb * kPlaneHalf + k4 * 2048), idesc_kv,
                                        (!first || term > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    // dK += dS^T Q_i
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            const int kk = 4 * hf + k4;
                            mma_ts_lead(leader, tmem + kColDK, tmem + kColDPT + 16 * kk + 8 * a,
                                        desc_advance(q_mn, bb * kPlaneHalf + k4 * 2048), idesc_kv,
                                        (!first || term > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    tc_commit_lead(leader, &sm.in_empty[slot]);
                    if (m == w.niter - 1 && hf == 1) tc_commit_lead(leader, &sm.grads_done);
                }
                if (!ok) break;
                // dQ_i = dS K_j over all 128 keys
                if (!mbar_wait_warp(&sm.ds_full, n & 1, ctx, SITE_DS_FULL)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    const int a = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; kk++) {
                        mma_ss_lead(leader, tmem + kColDQ, desc_advance(ds_mn[a], kk * 2048), desc_advance(k_mn[bb], kk * 2048),
                                    idesc_dq, (term > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                tc_commit_lead(leader, &sm.dq_full[n & 1]);
                if (m == w.niter - 1) tc_commit_lead(leader, &sm.k_free);
            }
            if (!feed.more) break;
        }
    }

    // ------------------------------ tear-down ------------------------------
    if (sm.abort_flag) __nanosleep(50000);  // let copies that are still in flight land
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(sm.tmem_base, kTmemCols);
    }
    // the last CTA to finish leaves the item counter as the next launch expects it
    if (threadIdx.x == 0 && atomicAdd(sched + 1, 1) == (int)gridDim.x - 1) {
        sched[0] = 0;
        sched[1] = 0;
    }
}

}  // namespace

static size_t bwd_smem_bytes() { return sizeof(BwdSmem); }
static_assert(sizeof(BwdSmem) <= 227 * 1024, "backward kernel shared memory");

cudaError_t fast_bwd_set_attributes() {
    return cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem_bytes());
}

// map_x / map_do must have boxes of 64 rows (see the producer warp); map_dx covers dqkv as fp32
// {3C, T, B} with boxes of 32 columns x 128 rows, 128-byte swizzle.  `num_sms` CTAs at most: one per SM,
// each taking (batch, head, key tile) items until none is left.  `sched` points at two ints that are zero
// when the kernel starts (the item counter and the number of CTAs that have finished) and zero again when
// it has completed.
cudaError_t launch_fast_backward(const CUtensorMap &map_x, const CUtensorMap &map_do, const CUtensorMap &map_dx,
                                 const float *lse, const float *delta, float *dqkv, int B, int T, int H, int num_sms,
                                 int *sched, int *status, cudaStream_t s) {
    const int nt = (T + kTile - 1) / kTile;
    const long long items = (long long)nt * B * H;
    if (items >= (long long)kMoreBit) return cudaErrorInvalidValue;  // an item number and a flag share one int
    const unsigned grid = (unsigned)(items < num_sms ? items : num_sms);
    const float scale = 0.125f;  // 1/sqrt(64)
    return launch_after_previous(attn_bwd_kernel, dim3(grid), dim3(kThreads), bwd_smem_bytes(), s, map_x, map_do, map_dx, lse,
                                 delta, dqkv, B, T, H, scale, scale * 1.4426950408889634f, sched, status);
}

}  // namespace attn
