// Fused causal attention forward for sm_100a, head size 64.
//
// Replaces attention_forward_cuda_kernel of gpt.c (kernels/src/cuda/Attention.cu:170-232): the
// permute kernel, the QK^T batched SGEMM, the mask and softmax kernels, the PV batched SGEMM and
// the unpermute kernel become one kernel that never writes the T x T matrix.
//
// One CTA handles one (batch, head) and one tile of 128 query rows, and walks the key tiles
// 0..diagonal.  Inputs are the bf16 hi/lo planes of the fused QKV tensor; Q/K/V tiles are
// addressed straight inside [B, T, 3C] by a 4-D tensor map (column, row, batch, plane).
//
// Warp roles (640 threads):
//   warp 0       TMA producer: Q once, then K tiles through a 2-stage ring
//   warp 3       TMA producer: V tiles through a 2-stage ring
//   warp 1       MMA issuer: S = Q K^T (SS, both K-major) and O_j = P V (P from tensor memory,
//                V MN-major from shared memory), each as hi*hi + hi*lo + lo*hi
//   warp 2       tensor-memory allocation / release
//   warps 4-11   softmax group 0: even key tiles
//   warps 12-19  softmax group 1: odd key tiles
// Each group's O accumulates in tensor memory across its tiles (the PV MMAs accumulate); the
// running reference maximum only moves when a row maximum exceeds it by more than 2^8, and only
// then is the accumulator rescaled in place.
// Inside a group two threads share a query row: warp quarter (warp % 4) selects the 32 rows the
// warp may touch in tensor memory, the warp half selects 64 of the 128 score columns and 32 of
// the 64 output columns.  The two halves exchange their row maximum through shared memory.
// Each group keeps its own running (max, sum, O) over its tiles; the two partial results are
// merged once at the end.  While one group works on S_j the tensor cores already compute
// S_{j+1} for the other group.
//
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) S2 [256,384) O0 [384,448) O1 [448,512).
// Three score buffers let the tensor cores run two key tiles ahead of the PV products, so a
// group that finishes a tile finds its next S already computed.
// P overwrites its own S buffer in place: each run of 16 score columns becomes 8 columns of
// packed bf16 hi parts followed by 8 columns of packed lo parts.
#include "attn_internal.h"
#include "tc05.cuh"

namespace attn {
namespace {

using namespace tc05;

constexpr int kTile = 128;
constexpr int kD = 64;
constexpr int kPlaneTile = kTile * kD * 2;  // bytes of one bf16 plane of a tile (16 KiB)
constexpr int kThreads = 640;
constexpr int kGroupThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 384;
constexpr int kSBufs = 3;
constexpr int kMergeStride = 65;  // floats per row of the merge buffer (odd: conflict free)

struct __align__(1024) FwdSmem {
    uint8_t q[2][kPlaneTile];     // [plane]
    uint8_t k[2][2][kPlaneTile];  // [stage][plane]
    uint8_t v[2][2][kPlaneTile];
    uint64_t q_full;
    uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t s_full[kSBufs], p_full[kSBufs], o_full[2];
    uint64_t pair_bar[2][4];  // [group][quarter]: the two halves of a row block meet here once per tile
    float xmax[2][2][2][kTile];  // [group][tile parity][half][row]: row maxima exchanged between halves
    float merge_l[2][2][kTile];  // [group][half][row]
    float merge_m[kTile];        // group 1's running maximum
    uint32_t tmem_base;
    int abort_flag;
};

enum Site : int {
    SITE_K_EMPTY = 1, SITE_V_EMPTY, SITE_Q_FULL, SITE_K_FULL, SITE_V_FULL, SITE_P_FULL, SITE_S_FULL, SITE_O_FULL,
    SITE_O_FULL_LAST, SITE_PAIR, SITE_MMA_IDLE
};

// Optional cycle trace of CTA 0 (debug builds with -DATTN_TRACE only).
#ifdef ATTN_TRACE
__device__ long long g_fwd_trace[3 * 16 * 8];
#define FWD_TRACE(cond, role, tile, k)                                                              \
    do {                                                                                            \
        if (blockIdx.x == 0 && (cond)) g_fwd_trace[((role) * 16 + (tile)) * 8 + (k)] = clock64();  \
    } while (0)
#else
#define FWD_TRACE(cond, role, tile, k) \
    do {                               \
    } while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Rescale threshold of the running reference maximum, in log2 units: the reference only moves
// when a tile's row maximum exceeds it by more than this, so P stays below 2^8 and the O
// accumulator in tensor memory rarely needs rescaling after a group's first tile.
constexpr float kRescaleThreshold = 8.0f;

// Max pass of one key tile of one softmax group.  kDiag: the tile on the diagonal needs the
// causal mask.  On return `alpha` is the factor by which the group's O accumulator must be
// rescaled before the PV product of this tile (1 when the reference maximum did not move).
// Returns false when the bounded wait on the partner half ran out.
template <bool kDiag>
__device__ __forceinline__ bool max_pass(FwdSmem &sm, const WaitCtx &ctx, uint32_t t_s, int row, int half, int wg,
                                         int par, uint64_t *pair_bar, float scale_log2, float &m, float &alpha) {
    uint32_t r0[32], r1[32];
    tmem_ld32(t_s + 64 * half, r0);
    tmem_ld32(t_s + 64 * half + 32, r1);
    tmem_wait_ld();
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        float a0 = __uint_as_float(r0[e]), a1 = __uint_as_float(r0[e + 1]);
        float b0 = __uint_as_float(r1[e]), b1 = __uint_as_float(r1[e + 1]);
        if (kDiag) {
            if (64 * half + e > row) a0 = -INFINITY;
            if (64 * half + e + 1 > row) a1 = -INFINITY;
            if (64 * half + 32 + e > row) b0 = -INFINITY;
            if (64 * half + 32 + e + 1 > row) b1 = -INFINITY;
        }
        mx = max3(mx, a0, a1);
        mx = max3(mx, b0, b1);
    }
    sm.xmax[wg][par][half][row] = mx;
    mbar_arrive(pair_bar);
    if (!mbar_wait_warp(pair_bar, par, ctx, SITE_PAIR)) return false;
    mx = fmaxf(mx, sm.xmax[wg][par][half ^ 1][row]) * scale_log2;
    const bool move = mx > m + kRescaleThreshold;  // always true on the first tile (m = -inf)
    alpha = move ? ex2(m - mx) : 1.0f;
    m = move ? mx : m;
    return true;
}

// exp pass: P = exp2(s * c - m), written over S in place as packed bf16 hi / lo.  The loads of
// the next 16 columns are in flight while the current 16 are processed.
// Returns this thread's partial row sum.
template <bool kDiag>
__device__ __forceinline__ float exp_pass(uint32_t t_s, int row, int half, float scale_log2, float m) {
    float2 lsum = make_float2(0.f, 0.f);
    const float2 sc2 = make_float2(scale_log2, scale_log2), mneg2 = make_float2(-m, -m);
    uint32_t r[2][16];
    tmem_ld16(t_s + 64 * half, r[0]);
#pragma unroll
    for (int c = 0; c < 4; c++) {
        tmem_wait_ld();
        if (c < 3) tmem_ld16(t_s + 64 * half + 16 * (c + 1), r[(c + 1) & 1]);
        const uint32_t col = 64 * half + 16 * c;
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float2 x = fma2(make_float2(__uint_as_float(r[c & 1][2 * e]), __uint_as_float(r[c & 1][2 * e + 1])),
                                  sc2, mneg2);
            float2 p = make_float2(ex2(x.x), ex2(x.y));
            if (kDiag) {
                if ((int)col + 2 * e > row) p.x = 0.f;
                if ((int)col + 2 * e + 1 > row) p.y = 0.f;
            }
            lsum = add2(lsum, p);
            split_bf16x2_packed(p, hi[e], lo[e]);
        }
        tmem_st8(t_s + col, hi);
        tmem_st8(t_s + col + 8, lo);
    }
    return lsum.x + lsum.y;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_x, float *__restrict__ out, float *__restrict__ out_copy,
                float *__restrict__ lse, int B, int T, int H, float scale_log2, int *status) {
    extern __shared__ uint8_t smem_raw[];
    FwdSmem &sm = *reinterpret_cast<FwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = B * H;
    const int nqt = (T + kTile - 1) / kTile;
    const int qt = nqt - 1 - (int)(blockIdx.x / BH);  // heaviest query tiles first
    const int bh = (int)(blockIdx.x % BH);
    const int b = bh / H, h = bh % H;
    const int C = H * kD;
    const int ntiles = qt + 1;  // key tiles 0..qt

    WaitCtx ctx{&sm.abort_flag, status};

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm.k_full[i], 1);
            mbar_init(&sm.k_empty[i], 1);
            mbar_init(&sm.v_full[i], 1);
            mbar_init(&sm.v_empty[i], 1);
            mbar_init(&sm.o_full[i], 1);
            for (int qd = 0; qd < 4; qd++) mbar_init(&sm.pair_bar[i][qd], 64);
        }
        for (int i = 0; i < kSBufs; i++) {
            mbar_init(&sm.s_full[i], 1);
            mbar_init(&sm.p_full[i], kGroupThreads);
        }
        fence_barrier_init();
    }
    if (warp == 2) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_x);
            const int xq = h * kD, xk = C + h * kD;
            mbar_expect_tx(&sm.q_full, 2 * kPlaneTile);
            tma_load_4d(sm.q[0], &map_x, &sm.q_full, xq, qt * kTile, b, 0);
            tma_load_4d(sm.q[1], &map_x, &sm.q_full, xq, qt * kTile, b, 1);
            for (int j = 0; j < ntiles; j++) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&sm.k_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_K_EMPTY)) break;
                mbar_expect_tx(&sm.k_full[st], 2 * kPlaneTile);
                tma_load_4d(sm.k[st][0], &map_x, &sm.k_full[st], xk, j * kTile, b, 0);
                tma_load_4d(sm.k[st][1], &map_x, &sm.k_full[st], xk, j * kTile, b, 1);
            }
        }
    } else if (warp == 3) {
        // ------------------------------ TMA producer for V ------------------------------
        // separate from the K producer: the K ring runs two tiles ahead of the V ring
        if (lane == 0) {
            const int xv = 2 * C + h * kD;
            for (int j = 0; j < ntiles; j++) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&sm.v_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_V_EMPTY)) break;
                mbar_expect_tx(&sm.v_full[st], 2 * kPlaneTile);
                tma_load_4d(sm.v[st][0], &map_x, &sm.v_full[st], xv, j * kTile, b, 0);
                tma_load_4d(sm.v[st][1], &map_x, &sm.v_full[st], xv, j * kTile, b, 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        {
            constexpr uint32_t idesc_s = idesc_bf16_f32(kTile, kTile, 0, 0);
            constexpr uint32_t idesc_o = idesc_bf16_f32(kTile, kD, 0, 1);
            const uint64_t qd[2] = {smem_desc_sw128(smem_u32(sm.q[0]), 16, 1024),
                                    smem_desc_sw128(smem_u32(sm.q[1]), 16, 1024)};
            bool ok = mbar_wait_warp(&sm.q_full, 0, ctx, SITE_Q_FULL);
            // Whichever product is ready goes next: S_j as soon as K_j has landed and a score
            // buffer is free (at most kSBufs tiles ahead of the PV products), O_j as soon as P_j
            // is published and V_j has landed.  S has priority: the softmax groups wait on it.
            int next_qk = 0, next_pv = 0;
            uint64_t idle_since = 0;
            uint32_t idle_polls = 0;
            while (ok && next_pv < ntiles) {
                bool progressed = false;
                if (next_qk < ntiles && next_qk - next_pv < kSBufs) {
                    const int j = next_qk, st = j & 1, buf = j % kSBufs;
                    if (__all_sync(0xffffffffu, mbar_test_wait(&sm.k_full[st], (j >> 1) & 1))) {
                        tc_fence_after_sync();
                        FWD_TRACE(lane == 0, 0, j, 1);
                        const uint64_t kd[2] = {smem_desc_sw128(smem_u32(sm.k[st][0]), 16, 1024),
                                                smem_desc_sw128(smem_u32(sm.k[st][1]), 16, 1024)};
                        const uint32_t d_s = tmem + kColS + buf * kTile;
                        uint32_t acc = 0;
#pragma unroll
                        for (int term = 0; term < 3; term++) {
                            const int qa = term == 2 ? 1 : 0, kb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                            for (int kk = 0; kk < kD / 16; kk++) {
                                mma_ss_elect(d_s, desc_advance(qd[qa], kk * 32), desc_advance(kd[kb], kk * 32),
                                             idesc_s, acc);
                                acc = 1;
                            }
                        }
                        tc_commit_elect(&sm.s_full[buf]);
                        tc_commit_elect(&sm.k_empty[st]);
                        FWD_TRACE(lane == 0, 0, j, 2);
                        next_qk++;
                        progressed = true;
                    }
                }
                if (next_pv < next_qk) {
                    const int jj = next_pv, st = jj & 1, buf = jj % kSBufs, ob = jj & 1;
                    if (__all_sync(0xffffffffu, mbar_test_wait(&sm.p_full[buf], (jj / kSBufs) & 1) &&
                                                    mbar_test_wait(&sm.v_full[st], (jj >> 1) & 1))) {
                        tc_fence_after_sync();
                        FWD_TRACE(lane == 0, 0, jj, 3);
                        const uint64_t vd[2] = {smem_desc_sw128(smem_u32(sm.v[st][0]), 1024, 1024),
                                                smem_desc_sw128(smem_u32(sm.v[st][1]), 1024, 1024)};
                        const uint32_t d_o = tmem + kColO + ob * kD;
                        const uint32_t p_base = tmem + kColS + buf * kTile;
                        uint32_t acc = jj >= 2 ? 1u : 0u;  // a group's O accumulates over its tiles
#pragma unroll
                        for (int term = 0; term < 3; term++) {
                            const int pa = term == 2 ? 1 : 0, vb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                            for (int kk = 0; kk < kTile / 16; kk++) {
                                mma_ts_elect(d_o, p_base + 16 * kk + 8 * pa, desc_advance(vd[vb], kk * 2048), idesc_o,
                                             acc);
                                acc = 1;
                            }
                        }
                        tc_commit_elect(&sm.o_full[ob]);
                        tc_commit_elect(&sm.v_empty[st]);
                        FWD_TRACE(lane == 0, 0, jj, 4);
                        next_pv++;
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
    } else if (warp >= 4) {
        // ------------------------------ softmax groups ------------------------------
        const int wg = (warp - 4) >> 3;            // 0: even tiles, 1: odd tiles
        const int half = ((warp - 4) >> 2) & 1;    // which 64 score columns / 32 output columns
        const int quarter = warp & 3;              // TMEM lane quarter this warp may access
        const int row = (quarter << 5) | lane;     // query row inside the tile == TMEM lane
        uint64_t *pair_bar = &sm.pair_bar[wg][quarter];
        const uint32_t lane_addr = (uint32_t)(quarter << 5) << 16;
        const uint32_t t_o = tmem + lane_addr + kColO + wg * kD + 32 * half;

        float m = -INFINITY, l = 0.f;
        bool pending = false, ok = true;
        int last_j = 0;

        for (int j = wg; j < ntiles; j += 2) {
            const int par = (j >> 1) & 1;
            FWD_TRACE(lane == 0 && half == 0 && quarter == 0, 1 + wg, j, 0);
            const int sb = j % kSBufs;
            const uint32_t t_s = tmem + lane_addr + kColS + sb * kTile;
            if (!mbar_wait_warp(&sm.s_full[sb], (j / kSBufs) & 1, ctx, SITE_S_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            FWD_TRACE(lane == 0 && half == 0 && quarter == 0, 1 + wg, j, 1);
            float alpha;
            const bool tile_ok = (j == qt)
                ? max_pass<true>(sm, ctx, t_s, row, half, wg, par, pair_bar, scale_log2, m, alpha)
                : max_pass<false>(sm, ctx, t_s, row, half, wg, par, pair_bar, scale_log2, m, alpha);
            if (!tile_ok) { ok = false; break; }
            FWD_TRACE(lane == 0 && half == 0 && quarter == 0, 1 + wg, j, 2);
            // The group's O accumulates in tensor memory over its tiles.  When the reference
            // maximum of some row of this warp moved, rescale the warp's 32 rows x 32 columns
            // of O in place: after the previous PV product has finished, before P_j is published.
            if (pending && __any_sync(0xffffffffu, alpha != 1.0f)) {
                if (!mbar_wait_warp(&sm.o_full[wg], ((j - 2) >> 1) & 1, ctx, SITE_O_FULL)) { ok = false; break; }
                tc_fence_after_sync();
                uint32_t r[32];
                tmem_ld32(t_o, r);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                tmem_st32(t_o, r);
            }
            l = l * alpha + ((j == qt) ? exp_pass<true>(t_s, row, half, scale_log2, m)
                                       : exp_pass<false>(t_s, row, half, scale_log2, m));
            FWD_TRACE(lane == 0 && half == 0 && quarter == 0, 1 + wg, j, 5);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_full[sb]);
            FWD_TRACE(lane == 0 && half == 0 && quarter == 0, 1 + wg, j, 6);
            pending = true;
            last_j = j;
        }
        float oacc[32];
#pragma unroll
        for (int d = 0; d < 32; d++) oacc[d] = 0.f;
        if (ok && pending) {
            if (mbar_wait_warp(&sm.o_full[wg], (last_j >> 1) & 1, ctx, SITE_O_FULL_LAST)) {
                tc_fence_after_sync();
                uint32_t r[32];
                tmem_ld32(t_o, r);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e++) oacc[e] = __uint_as_float(r[e]);
            } else {
                ok = false;
            }
        }

        // merge the two groups: everybody publishes its partial row sum, group 1 also its
        // maximum and O; group 0 combines and stores.  The K ring is idle by now (every QK^T
        // MMA precedes the last PV MMA of either group).
        float *merge_o = reinterpret_cast<float *>(sm.k);
        const bool has1 = ntiles >= 2;
        sm.merge_l[wg][half][row] = l;
        if (wg == 1 && has1 && ok) {
            if (half == 0) sm.merge_m[row] = m;
#pragma unroll
            for (int d = 0; d < 32; d++) merge_o[row * kMergeStride + 32 * half + d] = oacc[d];
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (wg == 0 && ok && !sm.abort_flag) {
            const float l0 = sm.merge_l[0][0][row] + sm.merge_l[0][1][row];
            float a0 = 1.f, a1 = 0.f, m_all = m, l_all = l0;
            if (has1) {
                const float m1 = sm.merge_m[row];
                const float l1 = sm.merge_l[1][0][row] + sm.merge_l[1][1][row];
                m_all = fmaxf(m, m1);
                a0 = ex2(m - m_all);
                a1 = ex2(m1 - m_all);
                l_all = l0 * a0 + l1 * a1;
            }
            const float inv = 1.0f / l_all;
            const int t = qt * kTile + row;
            if (t < T) {
                const size_t o_off = ((size_t)b * T + t) * C + (size_t)h * kD + 32 * half;
                float4 *dst = reinterpret_cast<float4 *>(out + o_off);
                float4 *dst2 = out_copy ? reinterpret_cast<float4 *>(out_copy + o_off) : nullptr;
#pragma unroll
                for (int d4 = 0; d4 < 8; d4++) {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float o = oacc[4 * d4 + e] * a0;
                        if (has1) o = fmaf(merge_o[row * kMergeStride + 32 * half + 4 * d4 + e], a1, o);
                        v[e] = o * inv;
                    }
                    const float4 f = make_float4(v[0], v[1], v[2], v[3]);
                    dst[d4] = f;
                    if (dst2) dst2[d4] = f;
                }
                if (half == 0) lse[(size_t)bh * T + t] = (m_all + __log2f(l_all)) * 0.6931471805599453f;
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    if (sm.abort_flag) __nanosleep(50000);  // let copies that are still in flight land
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

#ifdef ATTN_TRACE
extern "C" int attn_fwd_trace_read(long long *dst) {
    return (int)cudaMemcpyFromSymbol(dst, g_fwd_trace, sizeof(g_fwd_trace));
}
#endif

static size_t fwd_smem_bytes() { return sizeof(FwdSmem) + 1024; }

cudaError_t fast_fwd_set_attributes() {
    return cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem_bytes());
}

cudaError_t launch_fast_forward(const CUtensorMap &map_x, float *out, float *out_copy, float *lse, int B, int T, int H,
                                int *status, cudaStream_t s) {
    const int nqt = (T + kTile - 1) / kTile;
    const unsigned grid = (unsigned)(nqt * B * H);
    const float scale_log2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    attn_fwd_kernel<<<grid, kThreads, fwd_smem_bytes(), s>>>(map_x, out, out_copy, lse, B, T, H, scale_log2, status);
    return cudaGetLastError();
}

}  // namespace attn
