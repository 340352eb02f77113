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
// Warp roles (384 threads):
//   warp 0      TMA producer: Q once, then K and V tiles through 2-stage rings
//   warp 1      MMA issuer: S = Q K^T (SS, both K-major) and O_j = P V (P from tensor memory,
//               V MN-major from shared memory), each as hi*hi + hi*lo + lo*hi
//   warp 2      tensor-memory allocation / release
//   warps 4-7   softmax group 0: even key tiles      } one thread per query row; row max and
//   warps 8-11  softmax group 1: odd key tiles       } row sum need no shuffles in this layout
// Each softmax group keeps its own running (max, sum, O) over its tiles; the two partial
// results are merged once at the end.  While one group works on S_j the tensor cores already
// compute S_{j+1} for the other group.
//
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384).
// P overwrites its own S buffer: for each chunk of 32 score columns, columns [0,16) of the
// chunk receive the packed bf16 hi parts and columns [16,32) the lo parts.
#include "attn_internal.h"
#include "tc05.cuh"

namespace attn {
namespace {

using namespace tc05;

constexpr int kTile = 128;
constexpr int kD = 64;
constexpr int kPlaneTile = kTile * kD * 2;  // bytes of one bf16 plane of a tile (16 KiB)
constexpr int kThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;
constexpr int kMergeStride = 65;  // floats per row of the merge buffer (odd: conflict free)

struct __align__(1024) FwdSmem {
    uint8_t q[2][kPlaneTile];     // [plane]
    uint8_t k[2][2][kPlaneTile];  // [stage][plane]
    uint8_t v[2][2][kPlaneTile];
    uint64_t q_full;
    uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t s_full[2], p_full[2], o_full[2];
    float merge_ml[2][kTile];
    uint32_t tmem_base;
    int abort_flag;
};

enum Site : int {
    SITE_K_EMPTY = 1, SITE_V_EMPTY, SITE_Q_FULL, SITE_K_FULL, SITE_V_FULL, SITE_P_FULL, SITE_S_FULL, SITE_O_FULL,
    SITE_O_FULL_LAST
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
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
            mbar_init(&sm.s_full[i], 1);
            mbar_init(&sm.p_full[i], 128);
            mbar_init(&sm.o_full[i], 1);
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
            const int xq = h * kD, xk = C + h * kD, xv = 2 * C + h * kD;
            mbar_expect_tx(&sm.q_full, 2 * kPlaneTile);
            tma_load_4d(sm.q[0], &map_x, &sm.q_full, xq, qt * kTile, b, 0);
            tma_load_4d(sm.q[1], &map_x, &sm.q_full, xq, qt * kTile, b, 1);
            for (int j = 0; j < ntiles; j++) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait(&sm.k_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_K_EMPTY)) break;
                mbar_expect_tx(&sm.k_full[st], 2 * kPlaneTile);
                tma_load_4d(sm.k[st][0], &map_x, &sm.k_full[st], xk, j * kTile, b, 0);
                tma_load_4d(sm.k[st][1], &map_x, &sm.k_full[st], xk, j * kTile, b, 1);
                if (j >= 2 && !mbar_wait(&sm.v_empty[st], ((j >> 1) - 1) & 1, ctx, SITE_V_EMPTY)) break;
                mbar_expect_tx(&sm.v_full[st], 2 * kPlaneTile);
                tma_load_4d(sm.v[st][0], &map_x, &sm.v_full[st], xv, j * kTile, b, 0);
                tma_load_4d(sm.v[st][1], &map_x, &sm.v_full[st], xv, j * kTile, b, 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16_f32(kTile, kTile, 0, 0);
            constexpr uint32_t idesc_o = idesc_bf16_f32(kTile, kD, 0, 1);
            const uint64_t qd[2] = {smem_desc_sw128(smem_u32(sm.q[0]), 16, 1024),
                                    smem_desc_sw128(smem_u32(sm.q[1]), 16, 1024)};
            bool ok = mbar_wait(&sm.q_full, 0, ctx, SITE_Q_FULL);
            for (int j = 0; ok && j <= ntiles; j++) {
                if (j < ntiles) {
                    const int st = j & 1, buf = j & 1;
                    if (!mbar_wait(&sm.k_full[st], (j >> 1) & 1, ctx, SITE_K_FULL)) break;
                    tc_fence_after_sync();
                    const uint64_t kd[2] = {smem_desc_sw128(smem_u32(sm.k[st][0]), 16, 1024),
                                            smem_desc_sw128(smem_u32(sm.k[st][1]), 16, 1024)};
                    const uint32_t d_s = tmem + kColS + buf * kTile;
                    uint32_t acc = 0;
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int qa = term == 2 ? 1 : 0, kb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                        for (int kk = 0; kk < kD / 16; kk++) {
                            mma_ss(d_s, desc_advance(qd[qa], kk * 32), desc_advance(kd[kb], kk * 32), idesc_s, acc);
                            acc = 1;
                        }
                    }
                    tc_commit(&sm.s_full[buf]);
                    tc_commit(&sm.k_empty[st]);
                }
                if (j >= 1) {
                    const int jj = j - 1, st = jj & 1, buf = jj & 1;
                    if (!mbar_wait(&sm.v_full[st], (jj >> 1) & 1, ctx, SITE_V_FULL)) break;
                    if (!mbar_wait(&sm.p_full[buf], (jj >> 1) & 1, ctx, SITE_P_FULL)) break;
                    tc_fence_after_sync();
                    const uint64_t vd[2] = {smem_desc_sw128(smem_u32(sm.v[st][0]), 1024, 1024),
                                            smem_desc_sw128(smem_u32(sm.v[st][1]), 1024, 1024)};
                    const uint32_t d_o = tmem + kColO + buf * kD;
                    const uint32_t p_base = tmem + kColS + buf * kTile;
                    uint32_t acc = 0;
#pragma unroll
                    for (int term = 0; term < 3; term++) {
                        const int pa = term == 2 ? 1 : 0, vb = term == 1 ? 1 : 0;  // hh, hl, lh
#pragma unroll
                        for (int kk = 0; kk < kTile / 16; kk++) {
                            const uint32_t a_t = p_base + 32 * (kk >> 1) + 16 * pa + 8 * (kk & 1);
                            mma_ts(d_o, a_t, desc_advance(vd[vb], kk * 2048), idesc_o, acc);
                            acc = 1;
                        }
                    }
                    tc_commit(&sm.o_full[buf]);
                    tc_commit(&sm.v_empty[st]);
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------ softmax groups ------------------------------
        const int wg = (warp - 4) >> 2;           // 0: even tiles, 1: odd tiles
        const int row = ((warp & 3) << 5) | lane;  // query row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)((warp & 3) << 5) << 16;
        const uint32_t t_s = tmem + lane_addr + kColS + wg * kTile;
        const uint32_t t_o = tmem + lane_addr + kColO + wg * kD;

        float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
        float oacc[kD];
#pragma unroll
        for (int d = 0; d < kD; d++) oacc[d] = 0.f;
        bool pending = false, ok = true;
        int last_j = 0;

        for (int j = wg; j < ntiles; j += 2) {
            const uint32_t par = (j >> 1) & 1;
            const bool diag = (j == qt);
            if (!mbar_wait_warp(&sm.s_full[wg], par, ctx, SITE_S_FULL)) { ok = false; break; }
            tc_fence_after_sync();

            // pass 1: row maximum of the scaled scores
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t r[32];
                tmem_ld32(t_s + 32 * c, r);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    float v = __uint_as_float(r[e]) * scale_log2;
                    if (diag && (32 * c + e > row)) v = -INFINITY;
                    mx = fmaxf(mx, v);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = ex2(m - m_new);

            // fold in the previous tile's O (relative to the previous maximum)
            if (pending) {
                if (!mbar_wait_warp(&sm.o_full[wg], ((j - 2) >> 1) & 1, ctx, SITE_O_FULL)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t r[32];
                    tmem_ld32(t_o + 32 * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; e++) oacc[32 * c + e] = fmaf(oacc[32 * c + e], alpha_prev, __uint_as_float(r[e]));
                }
            }
            alpha_prev = alpha;
            l *= alpha;
            m = m_new;

            // pass 2: P = exp2(s - m), written back over S as packed bf16 hi / lo
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t r[32];
                tmem_ld32(t_s + 32 * c, r);
                tmem_wait_ld();
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int e = 0; e < 16; e++) {
                    float p0 = ex2(fmaf(__uint_as_float(r[2 * e]), scale_log2, -m));
                    float p1 = ex2(fmaf(__uint_as_float(r[2 * e + 1]), scale_log2, -m));
                    if (diag) {
                        if (32 * c + 2 * e > row) p0 = 0.f;
                        if (32 * c + 2 * e + 1 > row) p1 = 0.f;
                    }
                    l += p0 + p1;
                    split_bf16x2(p0, p1, hi[e], lo[e]);
                }
                tmem_st16(t_s + 32 * c, hi);
                tmem_st16(t_s + 32 * c + 16, lo);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_full[wg]);
            pending = true;
            last_j = j;
        }
        if (ok && pending) {
            if (mbar_wait_warp(&sm.o_full[wg], (last_j >> 1) & 1, ctx, SITE_O_FULL_LAST)) {
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t r[32];
                    tmem_ld32(t_o + 32 * c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; e++) oacc[32 * c + e] = fmaf(oacc[32 * c + e], alpha_prev, __uint_as_float(r[e]));
                }
            } else {
                ok = false;
            }
        }

        // merge the two groups: group 1 publishes (m, l, O); group 0 combines and stores.
        // The K ring is idle by now (every QK^T MMA precedes the last PV MMA of either group).
        float *merge_o = reinterpret_cast<float *>(sm.k);
        const bool has1 = ntiles >= 2;
        if (wg == 1 && has1 && ok) {
            sm.merge_ml[0][row] = m;
            sm.merge_ml[1][row] = l;
#pragma unroll
            for (int d = 0; d < kD; d++) merge_o[row * kMergeStride + d] = oacc[d];
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (wg == 0 && ok && !sm.abort_flag) {
            float a0 = 1.f, a1 = 0.f, m_all = m, l_all = l;
            if (has1) {
                const float m1 = sm.merge_ml[0][row], l1 = sm.merge_ml[1][row];
                m_all = fmaxf(m, m1);
                a0 = ex2(m - m_all);
                a1 = ex2(m1 - m_all);
                l_all = l * a0 + l1 * a1;
            }
            const float inv = 1.0f / l_all;
            const int t = qt * kTile + row;
            if (t < T) {
                const size_t o_off = ((size_t)b * T + t) * C + (size_t)h * kD;
                float4 *dst = reinterpret_cast<float4 *>(out + o_off);
                float4 *dst2 = out_copy ? reinterpret_cast<float4 *>(out_copy + o_off) : nullptr;
#pragma unroll
                for (int d4 = 0; d4 < kD / 4; d4++) {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float o = oacc[4 * d4 + e] * a0;
                        if (has1) o = fmaf(merge_o[row * kMergeStride + 4 * d4 + e], a1, o);
                        v[e] = o * inv;
                    }
                    const float4 f = make_float4(v[0], v[1], v[2], v[3]);
                    dst[d4] = f;
                    if (dst2) dst2[d4] = f;
                }
                lse[(size_t)bh * T + t] = (m_all + __log2f(l_all)) * 0.6931471805599453f;
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

cudaError_t launch_fast_forward(const CUtensorMap &map_x, float *out, float *out_copy, float *lse, int B, int T, int H,
                                int *status, cudaStream_t s) {
    const int nqt = (T + kTile - 1) / kTile;
    const unsigned grid = (unsigned)(nqt * B * H);
    const float scale_log2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    attn_fwd_kernel<<<grid, kThreads, fwd_smem_bytes(), s>>>(map_x, out, out_copy, lse, B, T, H, scale_log2, status);
    return cudaGetLastError();
}

}  // namespace attn
