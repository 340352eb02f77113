// Fused causal attention forward for sm_100a, head size 64.
//
// Replaces attention_forward_cuda_kernel of gpt.c (kernels/src/cuda/Attention.cu:170-232): the
// permute kernel, the QK^T batched SGEMM, the mask and softmax kernels, the PV batched SGEMM and
// the unpermute kernel become one kernel that never writes the T x T matrix.
//
// One CTA handles one (batch, head) and one tile of 128 query rows, and walks the keys up to the
// diagonal in steps of 64.  Inputs are the bf16 hi/lo planes of the fused QKV tensor; Q/K/V tiles are
// addressed straight inside [B, T, 3C] by a 4-D tensor map (column, row, batch, plane).
//
// The CTA is deliberately small (about 100 KiB of shared memory, 256 columns of tensor memory,
// 384 threads) so that TWO CTAs share an SM.  Inside a CTA two score buffers alternate, so the
// tensor cores compute S of the next key step while the softmax warps work on the current one;
// the second CTA fills what is still left idle, including the prologue and epilogue.
//
// Warp roles (384 threads):
//   warp 0       TMA producer for Q (once) and K (two-stage ring)
//   warp 1       MMA issuer: S = Q K^T (Q from tensor memory, K K-major from shared memory) and O += P V (P from tensor memory,
//                V MN-major from shared memory), each as hi*hi + hi*lo + lo*hi; the whole warp
//                runs the loop, one elected lane issues
//   warp 2       tensor-memory allocation / release
//   warp 3       TMA producer for V (two-stage ring)
//   warps 4-11   softmax: two threads per query row.  The warp quarter (warp % 4) selects the 32
//                rows the warp may touch in tensor memory, the warp half selects 32 of the 64
//                score columns of a step and 32 of the 64 output columns; the halves exchange
//                their row maximum through shared memory.
//
// Tensor memory (256 columns): S0 [0,64), S1 [64,128), O [128,192), Q hi/lo [192,256) (the A operand
// of S = Q K^T, copied once from shared memory).  P overwrites S in place: each run of 16
// score columns becomes 8 columns of packed bf16 hi parts followed by 8 columns of packed lo
// parts.  O accumulates in tensor memory across key tiles (the PV MMAs accumulate); the running
// reference maximum only moves when a row maximum exceeds it by more than 2^8, and only then is
// the accumulator rescaled in place.
#include "attn_internal.h"
#include "tc05.cuh"

namespace attn {
namespace {

using namespace tc05;

constexpr int kTile = 128;  // query rows per CTA
constexpr int kStep = 64;   // keys per step
constexpr int kD = 64;
constexpr int kPlaneTile = kTile * kD * 2;  // bytes of one bf16 plane of the Q tile (16 KiB)
constexpr int kPlaneStep = kStep * kD * 2;  // bytes of one bf16 plane of a K / V step (8 KiB)
constexpr int kThreads = 384;
constexpr int kSoftmaxThreads = 256;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128, kColQ = 192;  // Q: hi plane [192,224), lo plane [224,256)

struct __align__(1024) FwdSmem {
    uint8_t q[2][kPlaneTile];  // [plane]
    uint8_t k[2][2][kPlaneStep];  // [stage][plane]
    uint8_t v[2][2][kPlaneStep];
    uint64_t q_full, q_tmem, k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t s_full[2], p_full[2], o_full;
    uint64_t o_done;            // the last PV product has completed
    uint64_t epi_bar;           // every softmax thread has staged its part of the output tile
    uint64_t pair_bar[4];       // [quarter]: the two halves of a row block meet here once per tile
    float xmax[2][2][kTile];    // [tile parity][half][row]: row maxima exchanged between halves
    float lpart[2][kTile];      // [half][row]: partial row sums for the epilogue
    uint32_t tmem_base;
    int abort_flag;
};

enum Site : int {
    SITE_K_EMPTY = 1, SITE_V_EMPTY, SITE_Q_FULL, SITE_K_FULL, SITE_V_FULL, SITE_P_FULL, SITE_S_FULL, SITE_O_FULL,
    SITE_O_FULL_LAST, SITE_PAIR, SITE_Q_TMEM, SITE_EPI_BAR
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Rescale threshold of the running reference maximum, in log2 units: the reference only moves
// when a tile's row maximum exceeds it by more than this, so P stays below 2^8 and the O
// accumulator in tensor memory rarely needs rescaling after the first tile.
constexpr float kRescaleThreshold = 8.0f;

// Max pass of one key step.  kDiag: a step that touches the diagonal needs the causal mask; key0
// is the index of the step's first key relative to the first query row of the tile.  On return
// `alpha` is the factor by which the O accumulator must be rescaled before the PV product of
// this tile (1 when the reference maximum did not move).
// Returns false when the bounded wait on the partner half ran out.
template <bool kDiag>
__device__ __forceinline__ bool max_pass(FwdSmem &sm, const WaitCtx &ctx, uint32_t t_s, int row, int half, int par,
                                         int key0, uint64_t *pair_bar, float scale_log2, float &m, float &alpha) {
    uint32_t r0[32];
    tmem_ld32(t_s + 32 * half, r0);
    tmem_wait_ld();
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        float a0 = __uint_as_float(r0[e]), a1 = __uint_as_float(r0[e + 1]);
        if (kDiag) {
            if (key0 + 32 * half + e > row) a0 = -INFINITY;
            if (key0 + 32 * half + e + 1 > row) a1 = -INFINITY;
        }
        mx = max3(mx, a0, a1);
    }
    sm.xmax[par][half][row] = mx;
    mbar_arrive(pair_bar);
    if (!mbar_wait_warp(pair_bar, par, ctx, SITE_PAIR)) return false;
    mx = fmaxf(mx, sm.xmax[par][half ^ 1][row]) * scale_log2;
    const bool move = mx > m + kRescaleThreshold;  // always true on the first tile (m = -inf)
    alpha = move ? ex2(m - mx) : 1.0f;
    m = move ? mx : m;
    return true;
}

// exp pass: P = exp2(s * c - m), written over S in place as packed bf16 hi / lo.  The loads of
// the next 16 columns are in flight while the current 16 are processed.
// Returns this thread's partial row sum.
template <bool kDiag>
__device__ __forceinline__ float exp_pass(uint32_t t_s, int row, int half, int key0, float scale_log2, float m) {
    float2 lsum = make_float2(0.f, 0.f);
    const float2 sc2 = make_float2(scale_log2, scale_log2), mneg2 = make_float2(-m, -m);
    uint32_t r[2][16];
    tmem_ld16(t_s + 32 * half, r[0]);
#pragma unroll
    for (int c = 0; c < 2; c++) {
        tmem_wait_ld();
        if (c < 1) tmem_ld16(t_s + 32 * half + 16, r[1]);
        const uint32_t col = 32 * half + 16 * c;
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float2 x = fma2(make_float2(__uint_as_float(r[c][2 * e]), __uint_as_float(r[c][2 * e + 1])), sc2, mneg2);
            float2 p = make_float2(ex2(x.x), ex2(x.y));
            if (kDiag) {
                if (key0 + (int)col + 2 * e > row) p.x = 0.f;
                if (key0 + (int)col + 2 * e + 1 > row) p.y = 0.f;
            }
            lsum = add2(lsum, p);
            split_bf16x2_packed(p, hi[e], lo[e]);
        }
        tmem_st8(t_s + col, hi);
        tmem_st8(t_s + col + 8, lo);
    }
    return lsum.x + lsum.y;
}

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_out,
                const __grid_constant__ CUtensorMap map_copy, int out_maps, float *__restrict__ out,
                float *__restrict__ out_copy, float *__restrict__ lse, int B, int T, int H, float scale_log2, int *status) {
    extern __shared__ uint8_t smem_raw[];
    FwdSmem &sm = *reinterpret_cast<FwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = B * H;
    const int nqt = (T + kTile - 1) / kTile;
    const int qt = nqt - 1 - (int)(blockIdx.x / BH);  // heaviest query tiles first
    const int bh = (int)(blockIdx.x % BH);
    const int b = bh / H, h = bh % H;
    const int C = H * kD;
    const int nsteps = 2 * (qt + 1);  // key steps of 64 up to the end of the diagonal tile

    WaitCtx ctx{&sm.abort_flag, status};
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        mbar_init(&sm.q_tmem, kSoftmaxThreads);
        for (int i = 0; i < 2; i++) {
            mbar_init(&sm.k_full[i], 1);
            mbar_init(&sm.k_empty[i], 1);
            mbar_init(&sm.v_full[i], 1);
            mbar_init(&sm.v_empty[i], 1);
            mbar_init(&sm.s_full[i], 1);
            mbar_init(&sm.p_full[i], kSoftmaxThreads);
        }
        mbar_init(&sm.o_full, 1);
        mbar_init(&sm.o_done, 1);
        mbar_init(&sm.epi_bar, kSoftmaxThreads);
        for (int i = 0; i < 4; i++) mbar_init(&sm.pair_bar[i], 64);
        fence_barrier_init();
        // This thread is also the Q/K producer: Q and the first two K steps are requested right
        // away, while the other warps are still setting up (but not before the kernel that wrote
        // them has completed).
        pdl_wait();
        fence_proxy_async_smem();
        tma_prefetch_desc(&map_x);
        const int xq = h * kD, xk = C + h * kD;
        mbar_expect_tx(&sm.q_full, 2 * kPlaneTile);
        for (int hf = 0; hf < 2; hf++) {  // the tensor map's box is 64 rows
            tma_load_4d(sm.q[0] + hf * kPlaneStep, &map_x, &sm.q_full, xq, qt * kTile + hf * kStep, b, 0);
            tma_load_4d(sm.q[1] + hf * kPlaneStep, &map_x, &sm.q_full, xq, qt * kTile + hf * kStep, b, 1);
        }
        for (int j = 0; j < 2; j++) {  // nsteps >= 2
            mbar_expect_tx(&sm.k_full[j], 2 * kPlaneStep);
            tma_load_4d(sm.k[j][0], &map_x, &sm.k_full[j], xk, j * kStep, b, 0);
            tma_load_4d(sm.k[j][1], &map_x, &sm.k_full[j], xk, j * kStep, b, 1);
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
        // ------------------------------ TMA producer: K ------------------------------
        if (lane == 0) {
            const int xk = C + h * kD;
            for (int j = 2; j < nsteps; j++) {  // steps 0 and 1 were requested during set-up
                const int st = j & 1;
                if (!mbar_wait(&sm.k_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_K_EMPTY)) break;
                mbar_expect_tx(&sm.k_full[st], 2 * kPlaneStep);
                tma_load_4d(sm.k[st][0], &map_x, &sm.k_full[st], xk, j * kStep, b, 0);
                tma_load_4d(sm.k[st][1], &map_x, &sm.k_full[st], xk, j * kStep, b, 1);
            }
        }
    } else if (warp == 3) {
        // ------------------------------ TMA producer: V ------------------------------
        if (lane == 0) {
            const int xv = 2 * C + h * kD;
            for (int j = 0; j < nsteps; j++) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&sm.v_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_V_EMPTY)) break;
                mbar_expect_tx(&sm.v_full[st], 2 * kPlaneStep);
                tma_load_4d(sm.v[st][0], &map_x, &sm.v_full[st], xv, j * kStep, b, 0);
                tma_load_4d(sm.v[st][1], &map_x, &sm.v_full[st], xv, j * kStep, b, 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        constexpr uint32_t idesc_s = idesc_bf16_f32(kTile, kStep, 0, 0);
        constexpr uint32_t idesc_o = idesc_bf16_f32(kTile, kD, 0, 1);
        // Q is the A operand of every S = Q K^T of this CTA: the softmax warps copy it once from
        // shared to tensor memory, which halves the shared-memory traffic of those MMAs
        const uint32_t leader = elect_leader();  // the one lane that issues every MMA and commit
        bool ok = mbar_wait_warp(&sm.q_tmem, 0, ctx, SITE_Q_TMEM);
        // S of step j+1 is issued before the wait for P of step j: the two score buffers alternate,
        // so the tensor cores work on the next scores while the softmax warps are busy.  S_{j+1}
        // overwrites P_{j-1}; the tensor pipe runs in issue order, so PV_{j-1} has read it by then.
        auto issue_qk = [&](int j) -> bool {
            const int st = j & 1;
            if (!mbar_wait_warp(&sm.k_full[st], (j >> 1) & 1, ctx, SITE_K_FULL)) return false;
            tc_fence_after_sync();
            const uint64_t kd[2] = {smem_desc_sw128(smem_u32(sm.k[st][0]), 16, 1024),
                                    smem_desc_sw128(smem_u32(sm.k[st][1]), 16, 1024)};
            uint32_t acc = 0;
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const int qa = term == 2 ? 1 : 0, kb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                for (int kk = 0; kk < kD / 16; kk++) {
                    mma_ts_lead(leader, tmem + kColS + st * kStep, tmem + kColQ + 32 * qa + 8 * kk, desc_advance(kd[kb], kk * 32),
                                 idesc_s, acc);
                    acc = 1;
                }
            }
            tc_commit_lead(leader, &sm.s_full[st]);
            tc_commit_lead(leader, &sm.k_empty[st]);
            return true;
        };
        if (ok) ok = issue_qk(0);
        for (int j = 0; ok && j < nsteps; j++) {
            const int st = j & 1;
            if (j + 1 < nsteps && !issue_qk(j + 1)) break;
            // O += P_j V_j
            if (!mbar_wait_warp(&sm.v_full[st], (j >> 1) & 1, ctx, SITE_V_FULL)) break;
            if (!mbar_wait_warp(&sm.p_full[st], (j >> 1) & 1, ctx, SITE_P_FULL)) break;
            tc_fence_after_sync();
            const uint64_t vd[2] = {smem_desc_sw128(smem_u32(sm.v[st][0]), 1024, 1024),
                                    smem_desc_sw128(smem_u32(sm.v[st][1]), 1024, 1024)};
            uint32_t acc = j >= 1 ? 1u : 0u;
#pragma unroll
            for (int term = 0; term < 3; term++) {
                const int pa = term == 2 ? 1 : 0, vb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                for (int kk = 0; kk < kStep / 16; kk++) {
                    mma_ts_lead(leader, tmem + kColO, tmem + kColS + st * kStep + 16 * kk + 8 * pa,
                                 desc_advance(vd[vb], kk * 2048), idesc_o, acc);
                    acc = 1;
                }
            }
            tc_commit_lead(leader, &sm.o_full);
            tc_commit_lead(leader, &sm.v_empty[st]);
            if (j == nsteps - 1) tc_commit_lead(leader, &sm.o_done);
        }
    } else if (warp >= 4) {
        // ------------------------------ softmax ------------------------------
        const int half = (warp - 4) >> 2;       // which 64 score columns / 32 output columns
        const int quarter = warp & 3;           // TMEM lane quarter this warp may access
        const int row = (quarter << 5) | lane;  // query row inside the tile == TMEM lane
        uint64_t *pair_bar = &sm.pair_bar[quarter];
        const uint32_t lane_addr = (uint32_t)(quarter << 5) << 16;
        const uint32_t t_o = tmem + lane_addr + kColO + 32 * half;

        float m = -INFINITY, l = 0.f;

        // copy this thread's Q row (half 0: hi plane, half 1: lo plane) from the swizzled shared
        // memory tile into tensor memory: 64 bf16 = 32 packed columns, lane = row
        if (mbar_wait_warp(&sm.q_full, 0, ctx, SITE_Q_FULL)) {
            const uint8_t *qrow = sm.q[half] + row * 128;
            uint32_t r[32];
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint4 v = *reinterpret_cast<const uint4 *>(qrow + ((c ^ (row & 7)) << 4));
                r[4 * c] = v.x;
                r[4 * c + 1] = v.y;
                r[4 * c + 2] = v.z;
                r[4 * c + 3] = v.w;
            }
            tmem_st32(tmem + lane_addr + kColQ + 32 * half, r);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.q_tmem);
        }
        bool ok = true;

        for (int j = 0; j < nsteps; j++) {
            const int st = j & 1, par = (j >> 1) & 1;
            const uint32_t t_s = tmem + lane_addr + kColS + st * kStep;
            const int key0 = j * kStep - qt * kTile;  // first key of the step relative to the tile's first row
            const bool diag = key0 + kStep - 1 > 0;   // some (row, key) pair of this step is above the diagonal
            if (!mbar_wait_warp(&sm.s_full[st], par, ctx, SITE_S_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            float alpha;
            const bool step_ok = diag
                ? max_pass<true>(sm, ctx, t_s, row, half, j & 1, key0, pair_bar, scale_log2, m, alpha)
                : max_pass<false>(sm, ctx, t_s, row, half, j & 1, key0, pair_bar, scale_log2, m, alpha);
            if (!step_ok) { ok = false; break; }
            // When the reference maximum of some row of this warp moved, rescale the warp's 32 rows x
            // 32 columns of O in place: after the previous PV product has finished, before P_j is
            // published.
            if (j >= 1 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                if (!mbar_wait_warp(&sm.o_full, (j - 1) & 1, ctx, SITE_O_FULL)) { ok = false; break; }
                tc_fence_after_sync();
                uint32_t r[32];
                tmem_ld32(t_o, r);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                tmem_st32(t_o, r);
            }
            l = l * alpha + (diag ? exp_pass<true>(t_s, row, half, key0, scale_log2, m)
                                  : exp_pass<false>(t_s, row, half, key0, scale_log2, m));
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_full[st]);
        }

        // epilogue: O / l for this thread's 32 columns, log-sum-exp by the first half
        sm.lpart[half][row] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // The last product has a barrier of its own: o_full completes once per key step and this thread has
        // not followed its phases, so a parity wait on it could not tell the last product from the one before
        // (with two key steps the first PV can still be running here).
        if (ok && mbar_wait_warp(&sm.o_done, 0, ctx, SITE_O_FULL_LAST)) {
            tc_fence_after_sync();
            uint32_t r[32];
            tmem_ld32(t_o, r);
            tmem_wait_ld();
            const float l_all = sm.lpart[0][row] + sm.lpart[1][row];
            const float inv = 1.0f / l_all;
            const int t = qt * kTile + row;
            if (t < T && half == 0) lse[(size_t)bh * T + t] = (m + __log2f(l_all)) * 0.6931471805599453f;
            if (out_maps > 0) {
                // The normalised tile leaves through the copy engine: this thread's 32 columns are one
                // 128-byte row of a [128 x 32] fp32 box, staged (16-byte chunks swizzled by row % 8) in
                // the space of the Q tile, which has been dead since Q went to tensor memory.  Rows
                // past the end of the sequence are dropped by the copy engine.
                uint8_t *base = sm.q[half] + row * 128;
#pragma unroll
                for (int d4 = 0; d4 < 8; d4++)
                    *reinterpret_cast<float4 *>(base + ((d4 ^ (row & 7)) << 4)) =
                        make_float4(__uint_as_float(r[4 * d4]) * inv, __uint_as_float(r[4 * d4 + 1]) * inv,
                                    __uint_as_float(r[4 * d4 + 2]) * inv, __uint_as_float(r[4 * d4 + 3]) * inv);
                fence_proxy_async_smem();
                mbar_arrive(&sm.epi_bar);
                if (threadIdx.x == 128 && mbar_wait(&sm.epi_bar, 0, ctx, SITE_EPI_BAR)) {
                    tma_store_3d(sm.q[0], &map_out, h * kD, qt * kTile, b);
                    tma_store_3d(sm.q[1], &map_out, h * kD + 32, qt * kTile, b);
                    if (out_maps > 1) {
                        tma_store_3d(sm.q[0], &map_copy, h * kD, qt * kTile, b);
                        tma_store_3d(sm.q[1], &map_copy, h * kD + 32, qt * kTile, b);
                    }
                    bulk_commit();
                    bulk_wait_read_all();  // shared memory must stay alive until the copies have read it
                }
            } else if (t < T) {
                const size_t o_off = ((size_t)b * T + t) * C + (size_t)h * kD + 32 * half;
                float4 *dst = reinterpret_cast<float4 *>(out + o_off);
                float4 *dst2 = out_copy ? reinterpret_cast<float4 *>(out_copy + o_off) : nullptr;
#pragma unroll
                for (int d4 = 0; d4 < 8; d4++) {
                    const float4 f = make_float4(__uint_as_float(r[4 * d4]) * inv, __uint_as_float(r[4 * d4 + 1]) * inv,
                                                 __uint_as_float(r[4 * d4 + 2]) * inv, __uint_as_float(r[4 * d4 + 3]) * inv);
                    dst[d4] = f;
                    if (dst2) dst2[d4] = f;
                }
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

static size_t fwd_smem_bytes() { return sizeof(FwdSmem) + 1024; }

cudaError_t fast_fwd_set_attributes() {
    return cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem_bytes());
}

// map_out / map_copy: fp32 {C, T, B} maps of out / out_copy with boxes of 32 columns x 128 rows and
// 128-byte swizzle; with map_out == nullptr the kernel writes out (and out_copy) with plain stores.
cudaError_t launch_fast_forward(const CUtensorMap &map_x, const CUtensorMap *map_out, const CUtensorMap *map_copy,
                                float *out, float *out_copy, float *lse, int B, int T, int H, int *status, cudaStream_t s) {
    const int nqt = (T + kTile - 1) / kTile;
    const unsigned grid = (unsigned)(nqt * B * H);
    const float scale_log2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    const int out_maps = map_out ? (map_copy && out_copy ? 2 : 1) : 0;
    const CUtensorMap &mo = map_out ? *map_out : map_x;  // unused by the kernel when out_maps == 0
    const CUtensorMap &mc = out_maps == 2 ? *map_copy : mo;
    return launch_after_previous(attn_fwd_kernel, dim3(grid), dim3(kThreads), fwd_smem_bytes(), s, map_x, mo, mc, out_maps, out,
                                 out_copy, lse, B, T, H, scale_log2, status);
}

}  // namespace attn
