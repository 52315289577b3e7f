// Split-K decode / speculative-verify attention over the paged Q8_0 KV cache, head_dim 128.
//
// Semantics: attn_decode_global_q8k (crates/sg-gpu/shaders/attn_decode_global_q8k.wgsl:18-112)
// extended with Q8_0 V, a page table and up to 4 query tokens.  Grid meaning, split ranges
// (chunk = ceil(kv_len / n_splits), l.52-54), the -3e38 sentinel for empty splits (l.68) and the
// partials layout part[(row * n_splits + split) * 130] = acc[128], m, l (l.101-111) are the
// reference's; row = i * H + qh for query token i.
//
// Design (HBM-bound: 17/16 byte per K/V element is all that has to move):
//   * one CTA per (kv head, split); a producer warp streams 64-token stages of K quants, K scales,
//     V quants, V scales with TMA into a ring of shared-memory stages (mbarrier full/empty pairs),
//     translating logical tokens through the page table once per stage;
//   * four consumer warps each own 16 tokens of a stage.  int8 bytes are turned into exact f16
//     integers straight out of shared memory with byte permutes (0x6400 | (q ^ 0x80) = q + 1152)
//     and fed to mma.sync m16n8k16 -- the tile is (8 query rows) x (16 tokens), far below the
//     64-row minimum of tcgen05, so the warp-level MMA is the right tool here;
//   * the per-block scales never touch the int8 data: QK^T is accumulated per 32-wide block and
//     multiplied by f32(scale) afterwards (sum_b s_b * sum_d q_d k_d == sum_d q_d (s_b k_d), i.e.
//     the reference's exact product f32(scale)*f32(q), no f16 re-rounding); for PV the scale is
//     folded into P.  The +1152 offsets are removed exactly: the QK accumulator starts at
//     -1152 * sum(q) and PV subtracts 1152 * sum(P') gathered by one extra MMA against ones;
//   * online softmax in registers (base-2, row max by warp shuffles over the 4 lanes of a row,
//     rescale only when the max grows by more than 2^8), warps merged in fixed order.
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <string>

#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int HD = 128;
constexpr int G = 2;                     // query heads per kv head
constexpr int STAGE_TOK = 64;            // tokens per pipeline stage
constexpr int CONSUMER_WARPS = 4;        // 16 tokens each
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int MAX_ROWS = 8;              // query rows in the MMA tile = m_q * G, m_q <= 4
constexpr uint32_t Q_TILE_BYTES = STAGE_TOK * 128;
constexpr uint32_t S_TILE_BYTES = STAGE_TOK * 16;
constexpr uint32_t STAGE_BYTES = 2 * Q_TILE_BYTES + 2 * S_TILE_BYTES;
constexpr uint32_t MAGIC = 0x64646464u;  // high byte of f16 1024.0
constexpr float OFFSET = 1152.0f;        // 1024 + 128
constexpr float RESCALE_T = 8.0f;        // lazy-rescale threshold, log2 units

template <int NSTAGES>
struct __align__(1024) DecodeSmem {
    uint8_t kq[NSTAGES][Q_TILE_BYTES];   // [64 tokens][128 B], 128-byte swizzled by TMA
    uint8_t vq[NSTAGES][Q_TILE_BYTES];
    uint8_t ks[NSTAGES][S_TILE_BYTES];   // [64 tokens][8 f16]: scales of a pair of kv heads
    uint8_t vs[NSTAGES][S_TILE_BYTES];
    float merge[CONSUMER_WARPS][MAX_ROWS][HD + 2];
    uint64_t full[NSTAGES];
    uint64_t empty[NSTAGES];
};

// mma.sync m16n8k16 with only the top 8 rows of A in use (rows 8..15 are zero).  The bottom half of
// the accumulator is then c2 = c3 = 0 in and out, so it gets constants in and throw-away registers
// out instead of live state: (c0, c1) is the accumulator of row g, columns 2*t4 and 2*t4 + 1.
__device__ __forceinline__ void mma_top(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1)
{
    float dead0, dead1;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%9,%9};"
        : "+f"(c0), "+f"(c1), "=f"(dead0), "=f"(dead1)
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ float quad_max(float v)
{
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int NSTAGES, int MIN_CTAS>
__global__ void __launch_bounds__(THREADS, MIN_CTAS) decode_paged_kernel(const __grid_constant__ CUtensorMap tm_kq,
                                                               const __grid_constant__ CUtensorMap tm_ks,
                                                               const __grid_constant__ CUtensorMap tm_vq,
                                                               const __grid_constant__ CUtensorMap tm_vs,
                                                               const __half* __restrict__ q,
                                                               const uint32_t* __restrict__ page_table, uint32_t table_len,
                                                               uint32_t page, uint32_t pool_pages, float* __restrict__ part,
                                                               const uint32_t* __restrict__ step, uint32_t n_splits,
                                                               float scale, uint32_t m_q, uint32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    using Smem = DecodeSmem<NSTAGES>;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.x, n_kv = gridDim.x, split = blockIdx.y;
    const int n_q = n_kv * G;

    const uint32_t kv_len = step[STEP_KV_LEN_GLOBAL];
    const uint32_t chunk = (kv_len + n_splits - 1) / n_splits;
    const uint32_t t_begin = min((uint32_t)split * chunk, kv_len);
    const uint32_t t_end = min(t_begin + chunk, kv_len);
    const uint32_t s_begin = t_begin / STAGE_TOK;
    const uint32_t n_iter = t_begin < t_end ? (t_end + STAGE_TOK - 1) / STAGE_TOK - s_begin : 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGES; i++) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_kq);
            tma_prefetch_desc(&tm_ks);
            tma_prefetch_desc(&tm_vq);
            tma_prefetch_desc(&tm_vs);
            bool failed = false;
            for (uint32_t it = 0; it < n_iter; ++it) {
                const int st = it % NSTAGES;
                const uint32_t round = it / NSTAGES;
                if (round > 0) mbar_wait(&sm.empty[st], (round - 1) & 1, status, 301, failed);
                if (failed) break;
                const uint32_t tok0 = (s_begin + it) * STAGE_TOK;
                const uint32_t lp = tok0 / page;
                uint32_t pp = 0;
                if (lp < table_len) {
                    pp = page_table[lp];
                } else {
                    report_error(status, DEV_ERR_BOUNDS, 302, lp, table_len);
                }
                if (pp >= pool_pages) {
                    report_error(status, DEV_ERR_BOUNDS, 303, pp, pool_pages);
                    pp = 0;
                }
                const int row = (int)(pp * page + tok0 % page);
                mbar_arrive_expect_tx(&sm.full[st], STAGE_BYTES);
                tma_load_3d(sm.kq[st], &tm_kq, &sm.full[st], 0, kvh, row);
                tma_load_2d(sm.ks[st], &tm_ks, &sm.full[st], (kvh >> 1) * 8, row);
                tma_load_3d(sm.vq[st], &tm_vq, &sm.full[st], 0, kvh, row);
                tma_load_2d(sm.vs[st], &tm_vs, &sm.full[st], (kvh >> 1) * 8, row);
            }
            // Do not leave with copies in flight: wait (bounded) for the last use of every stage.
            if (!failed) {
                const uint32_t first = n_iter > (uint32_t)NSTAGES ? n_iter - NSTAGES : 0;
                for (uint32_t it = first; it < n_iter; ++it)
                    mbar_wait(&sm.full[it % NSTAGES], (it / NSTAGES) & 1, status, 304, failed);
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2, t4 = lane & 3;
        const uint32_t rows = m_q * G;
        const bool row_live = (uint32_t)g < rows;
        const uint32_t qi = (uint32_t)g / G;
        const int qh = kvh * G + g % G;
        // Last key this row may see: kv_len - m_q + qi  (all of them when m_q == 1).
        const int64_t vis_last = (int64_t)kv_len - (int64_t)m_q + (int64_t)qi;

        // Q fragments of mma.m16n8k16 (A operand, rows = query rows; rows 8..15 are zero).  With the
        // K bytes of a 32-wide block split 8 per lane (lane t4 holds bytes 8*t4 .. 8*t4+7), k-step s
        // contracts dims 32b + 8*t4 + 4s + {0,1 | 2,3}.
        uint32_t qa[4][2][2];
        float cinit[4];
        {
            const __half* qrow = q + ((size_t)qi * n_q + qh) * HD;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                float sum = 0.0f;
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    uint2 w = make_uint2(0u, 0u);
                    if (row_live) w = __ldg(reinterpret_cast<const uint2*>(qrow + 32 * b + 8 * t4 + 4 * s));
                    qa[b][s][0] = w.x;
                    qa[b][s][1] = w.y;
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
                    sum += (f0.x + f0.y) + (f1.x + f1.y);
                }
                cinit[b] = -OFFSET * quad_sum(sum);
            }
        }

        const float scale2 = scale * 1.4426950408889634f;
        float m_run = NEG_SENTINEL, l_part = 0.0f;
        float o[4][4][2];   // [block][i]: c0 -> dim 32b + 8*t4 + i, c1 -> dim 32b + 8*t4 + 4 + i
        float osum[4];      // sum over tokens of P'_b for this row
#pragma unroll
        for (int b = 0; b < 4; b++) {
            osum[b] = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) o[b][i][0] = o[b][i][1] = 0.0f;
        }

        bool failed = false;
        for (uint32_t it = 0; it < n_iter; ++it) {
            const int st = it % NSTAGES;
            mbar_wait(&sm.full[st], (it / NSTAGES) & 1, status, 305, failed);
            const uint32_t tile_tok0 = (s_begin + it) * STAGE_TOK + 16 * warp;
            const int r0 = 16 * warp;  // first smem row of this warp's tile

            // ---- S^T = Q K^T per block: rows = query rows, columns = tokens --------------------
            float sacc[2][4][2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int row = r0 + 8 * j + g;  // the token this lane supplies as B column n = g
                const uint8_t* krow = sm.kq[st] + row * 128;
                const int swz = row & 7;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int c16 = (2 * b + (t4 >> 1)) ^ swz;
                    uint2 w = *reinterpret_cast<const uint2*>(krow + c16 * 16 + (t4 & 1) * 8);
                    w.x ^= 0x80808080u;
                    w.y ^= 0x80808080u;
                    sacc[j][b][0] = cinit[b];
                    sacc[j][b][1] = cinit[b];
                    mma_top(sacc[j][b][0], sacc[j][b][1], qa[b][0][0], qa[b][0][1], __byte_perm(w.x, MAGIC, 0x4140),
                            __byte_perm(w.x, MAGIC, 0x4342));
                    mma_top(sacc[j][b][0], sacc[j][b][1], qa[b][1][0], qa[b][1][1], __byte_perm(w.y, MAGIC, 0x4140),
                            __byte_perm(w.y, MAGIC, 0x4342));
                }
            }

            // ---- scores for this lane's 4 tokens: (j, e) -> token r0 + 8j + 2*t4 + e --------------
            float s2[2][2];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; j++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int tok = r0 + 8 * j + 2 * t4 + e;
                    const uint2 sw = *reinterpret_cast<const uint2*>(sm.ks[st] + tok * 16 + (kvh & 1) * 8);
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sw.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sw.y));
                    float s = s01.x * sacc[j][0][e];
                    s = fmaf(s01.y, sacc[j][1][e], s);
                    s = fmaf(s23.x, sacc[j][2][e], s);
                    s = fmaf(s23.y, sacc[j][3][e], s);
                    const int64_t T = (int64_t)tile_tok0 + 8 * j + 2 * t4 + e;
                    const bool vis = T >= (int64_t)t_begin && T < (int64_t)t_end && T <= vis_last;
                    s2[j][e] = vis ? s * scale2 : -INFINITY;
                    mx = fmaxf(mx, s2[j][e]);
                }
            }
            mx = quad_max(mx);
            const bool grow = mx > m_run + RESCALE_T;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? mx : m_run;
                const float corr = ex2(m_run - m_new);
                m_run = m_new;
                l_part *= corr;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    osum[b] *= corr;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        o[b][i][0] *= corr;
                        o[b][i][1] *= corr;
                    }
                }
            }
            float p[2][2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    p[j][e] = ex2(s2[j][e] - m_run);
                    l_part += p[j][e];
                }
            }

            // ---- O += P' V with P'_b = P * s_b(V): A rows = query rows, k = this tile's 16 tokens ---
            float sv[2][2][4];
#pragma unroll
            for (int j = 0; j < 2; j++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int tok = r0 + 8 * j + 2 * t4 + e;
                    const uint2 sw = *reinterpret_cast<const uint2*>(sm.vs[st] + tok * 16 + (kvh & 1) * 8);
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sw.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sw.y));
                    sv[j][e][0] = s01.x;
                    sv[j][e][1] = s01.y;
                    sv[j][e][2] = s23.x;
                    sv[j][e][3] = s23.y;
                }
            }
            const uint8_t* vbase = sm.vq[st];
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const uint32_t pa0 = pack_half2(p[0][0] * sv[0][0][b], p[0][1] * sv[0][1][b]);
                const uint32_t pa2 = pack_half2(p[1][0] * sv[1][0][b], p[1][1] * sv[1][1][b]);
                uint32_t w[2][2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int row = r0 + 8 * j + 2 * t4 + e;
                        const int c16 = (2 * b + (g >> 2)) ^ (row & 7);
                        w[j][e] = *reinterpret_cast<const uint32_t*>(vbase + row * 128 + c16 * 16 + (g & 3) * 4) ^ 0x80808080u;
                    }
                }
                // pair the two tokens of a k-slot byte by byte, then widen to f16
                const uint32_t lo0 = __byte_perm(w[0][0], w[0][1], 0x5140), hi0 = __byte_perm(w[0][0], w[0][1], 0x7362);
                const uint32_t lo1 = __byte_perm(w[1][0], w[1][1], 0x5140), hi1 = __byte_perm(w[1][0], w[1][1], 0x7362);
                mma_top(o[b][0][0], o[b][0][1], pa0, pa2, __byte_perm(lo0, MAGIC, 0x4140), __byte_perm(lo1, MAGIC, 0x4140));
                mma_top(o[b][1][0], o[b][1][1], pa0, pa2, __byte_perm(lo0, MAGIC, 0x4342), __byte_perm(lo1, MAGIC, 0x4342));
                mma_top(o[b][2][0], o[b][2][1], pa0, pa2, __byte_perm(hi0, MAGIC, 0x4140), __byte_perm(hi1, MAGIC, 0x4140));
                mma_top(o[b][3][0], o[b][3][1], pa0, pa2, __byte_perm(hi0, MAGIC, 0x4342), __byte_perm(hi1, MAGIC, 0x4342));
                float ones_c1 = 0.0f;  // every column of P' x ones is the row sum; keep column 2*t4 only
                mma_top(osum[b], ones_c1, pa0, pa2, 0x3C003C00u, 0x3C003C00u);
            }

            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[st]);
        }

        // ---- this warp's (acc, m, l) into shared memory ---------------------------------------
        const float l_row = quad_sum(l_part);
        if (g < MAX_ROWS) {
            float* dst = sm.merge[warp][g];
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const float corr = OFFSET * osum[b];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    dst[32 * b + 8 * t4 + i] = o[b][i][0] - corr;
                    dst[32 * b + 8 * t4 + 4 + i] = o[b][i][1] - corr;
                }
            }
            if (t4 == 0) {
                dst[HD] = m_run == NEG_SENTINEL ? NEG_SENTINEL : m_run * 0.6931471805599453f;  // back to natural log
                dst[HD + 1] = l_row;
            }
        }
    }
    __syncthreads();

    // ---- merge the four warps in fixed order and write the split's partial --------------------------
    if (threadIdx.x < CONSUMER_WARPS * 32) {
        const int row = threadIdx.x >> 4, d0 = (threadIdx.x & 15) * 8;
        if ((uint32_t)row < m_q * G) {
            float m_all = NEG_SENTINEL;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; w++) m_all = fmaxf(m_all, sm.merge[w][row][HD]);
            float acc[8], l = 0.0f;
#pragma unroll
            for (int d = 0; d < 8; d++) acc[d] = 0.0f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; w++) {
                const float f = __expf(sm.merge[w][row][HD] - m_all);
                l = fmaf(f, sm.merge[w][row][HD + 1], l);
#pragma unroll
                for (int d = 0; d < 8; d++) acc[d] = fmaf(f, sm.merge[w][row][d0 + d], acc[d]);
            }
            const uint32_t qi = (uint32_t)row / G;
            const int qh = kvh * G + row % G;
            float* dst = part + (((size_t)qi * n_q + qh) * n_splits + split) * (HD + 2);
#pragma unroll
            for (int d = 0; d < 8; d++) dst[d0 + d] = acc[d];
            if (d0 == 0) {
                dst[HD] = m_all;
                dst[HD + 1] = l;
            }
        }
    }
}

struct PushDecodePaged {
    uint32_t n_splits;
    float scale;
    uint32_t page;
};

template <int NSTAGES, int MIN_CTAS>
int launch_variant(const LaunchArgs& a, const CUtensorMap (&tm)[4], const PushDecodePaged& p, int n_kv, uint32_t m_q,
                   size_t pool_rows)
{
    using Smem = DecodeSmem<NSTAGES>;
    const size_t smem = sizeof(Smem) + 1024;
    static bool attr_set[64] = {};
    if (a.device < 64 && !attr_set[a.device]) {
        if (int r = check_cuda(a, cudaFuncSetAttribute(decode_paged_kernel<NSTAGES, MIN_CTAS>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                               "cudaFuncSetAttribute(decode_paged)"))
            return r;
        attr_set[a.device] = true;
    }
    decode_paged_kernel<NSTAGES, MIN_CTAS><<<dim3(n_kv, p.n_splits), THREADS, smem, a.stream>>>(
        tm[0], tm[1], tm[2], tm[3], (const __half*)a.b[0].ptr, (const uint32_t*)a.b[5].ptr, (uint32_t)(a.b[5].bytes / 4), p.page,
        (uint32_t)(pool_rows / p.page), (float*)a.b[6].ptr, (const uint32_t*)a.b[7].ptr, p.n_splits, p.scale, m_q, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_decode_paged_q8kv_d128");
}

// Pipeline shape: 3 stages x 18 KB + the merge buffer = 72 KB, three CTAs per SM (default), or
// 4 stages and two CTAs per SM with more registers per thread.  SGB_DECODE_PIPELINE=4x2 picks the
// second; it exists for tuning and changes no result bit.
int pipeline_choice()
{
    static int choice = [] {
        const char* e = getenv("SGB_DECODE_PIPELINE");
        return (e && e[0] == '4') ? 1 : 0;
    }();
    return choice;
}

}  // namespace

// attn_decode_paged_q8kv_d128 / attn_verify_paged_q8kv_d128.
// bindings: q f16 [m_q x H x 128], k_quants i8, k_scales f16, v_quants i8, v_scales f16,
//           page_table u32, part f32 [m_q*H x n_splits x 130], step.
// push {n_splits u32, scale f32, page u32}.  grid [n_kv_heads, n_splits, m_q (0 or 1 = decode)].
int launch_decode_paged_q8kv_d128(const LaunchArgs& a)
{
    const PushDecodePaged p = *(const PushDecodePaged*)a.push;
    const int n_kv = (int)a.groups[0];
    const uint32_t m_q = a.groups[2] ? a.groups[2] : 1;
    if (n_kv <= 0 || (n_kv & 1)) return fail_validation(a, "decode_paged: groups[0] (kv heads) must be even and > 0");
    if (p.n_splits == 0 || a.groups[1] != p.n_splits)
        return fail_validation(a, "decode_paged: groups[1] must equal push.n_splits (> 0)");
    if (m_q > 4) return fail_validation(a, "decode_paged: at most 4 query tokens");
    if (p.page == 0 || p.page % STAGE_TOK) return fail_validation(a, "decode_paged: page must be a multiple of 64 tokens");
    const size_t row_bytes = (size_t)n_kv * HD;
    const size_t pool_rows = a.b[1].bytes / row_bytes;
    if (pool_rows == 0 || a.b[3].bytes / row_bytes != pool_rows)
        return fail_validation(a, "decode_paged: K and V quant pools must hold the same (non-zero) number of rows");
    if (a.b[2].bytes / 2 < pool_rows * n_kv * 4 || a.b[4].bytes / 2 < pool_rows * n_kv * 4)
        return fail_validation(a, "decode_paged: scales pool too short for its quants pool");
    if (a.b[5].bytes < 4) return fail_validation(a, "decode_paged: empty page table");
    const size_t n_q = (size_t)n_kv * G;
    if (a.b[0].bytes < m_q * n_q * HD * 2) return fail_validation(a, "decode_paged: q buffer too small");
    if (int r = need_bytes(a, 6, m_q * n_q * p.n_splits * (HD + 2) * 4, "part")) return r;
    if (int r = need_bytes(a, 7, 16, "step")) return r;
    for (int i = 1; i <= 4; i++)
        if (reinterpret_cast<uintptr_t>(a.b[i].ptr) & 15) return fail_validation(a, "decode_paged: K/V pools must be 16-byte aligned");

    CUtensorMap tm[4];
    for (int i = 0; i < 2; i++) {
        const uint64_t qd[3] = {HD, (uint64_t)n_kv, pool_rows};
        const uint64_t qs[2] = {HD, row_bytes};
        const uint32_t qb[3] = {HD, 1, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i], 0, 3, a.b[1 + 2 * i].ptr, qd, qs, qb, 3)) return r;
        const uint64_t sd[2] = {(uint64_t)n_kv * 4, pool_rows};
        const uint64_t ss[1] = {(uint64_t)n_kv * 8};
        const uint32_t sb[2] = {8, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i + 1], 1, 2, a.b[2 + 2 * i].ptr, sd, ss, sb, 0)) return r;
    }

    return pipeline_choice() ? launch_variant<4, 2>(a, tm, p, n_kv, m_q, pool_rows)
                             : launch_variant<3, 3>(a, tm, p, n_kv, m_q, pool_rows);
}

}  // namespace sgb

// ====================================================================================================
// Allocation-free decode: sgb_decode_paged_q8kv_d128_noalloc
//
// Some hosts may not allocate device memory at the moment they need attention: a serving loop that
// has handed every byte of HBM to its KV pool, or code running between an allocator's bookkeeping
// phases where a cudaMalloc would stall the device.  This entry point does the whole decode step
// -- split-K partials and the log-sum-exp combine -- without allocating anything, on the device or
// through any library: the split-K partials and the four step words live in the file-scope array
// below, which every GPU that loads this library holds until the process exits (about 1.04 MB).
// ====================================================================================================
namespace sgb {
namespace {

constexpr uint32_t NOALLOC_MAX_PART_ROWS = 2048;  // (query rows) x (splits) the scratch can hold
constexpr size_t NOALLOC_PART_FLOATS = (size_t)NOALLOC_MAX_PART_ROWS * (HD + 2);
constexpr size_t NOALLOC_STEP_AT = NOALLOC_PART_FLOATS;  // 4 x u32 step words after the partials

static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_PART_FLOATS + 64];

// In host code `g_noalloc_scratch` is only a handle; the device address comes from
// cudaGetSymbolAddress, once per device.
void* g_noalloc_dev_ptr[64] = {};
bool g_noalloc_ready[64] = {};

__global__ void noalloc_step_kernel(uint32_t kv_len)
{
    uint32_t* step = reinterpret_cast<uint32_t*>(g_noalloc_scratch + NOALLOC_STEP_AT);
    step[STEP_POS] = 0;
    step[STEP_KV_LEN_SLIDING] = 0;
    step[STEP_KV_LEN_GLOBAL] = kv_len;
    step[STEP_Q0] = 0;
}

// Combine of the splits in ascending order (the arithmetic of attn_reduce.wgsl:29-56), reading the
// partials straight from the static array.  One block per query row, one thread per dim.
__global__ void __launch_bounds__(HD) noalloc_reduce_kernel(float* __restrict__ out, uint32_t n_splits)
{
    const size_t row = blockIdx.x;
    const int d = threadIdx.x;
    float m = NEG_SENTINEL, l = 0.0f, acc = 0.0f;
    for (uint32_t s = 0; s < n_splits; s++) {
        const float* p = g_noalloc_scratch + (row * n_splits + s) * (HD + 2);
        const float ms = p[HD], ls = p[HD + 1];
        const float m_new = fmaxf(m, ms);
        const float ca = __expf(m - m_new), cb = __expf(ms - m_new);
        acc = acc * ca + p[d] * cb;
        l = l * ca + ls * cb;
        m = m_new;
    }
    out[row * HD + d] = acc / l;
}

}  // namespace
}  // namespace sgb

extern "C" int sgb_decode_paged_q8kv_d128_noalloc(int device, void* stream, const void* q, const void* k_quants,
                                                  const void* k_scales, const void* v_quants, const void* v_scales,
                                                  const uint32_t* page_table, uint32_t table_len, uint64_t pool_rows,
                                                  float* out, uint32_t* status, uint32_t n_kv_heads, uint32_t m_q,
                                                  uint32_t kv_len, uint32_t n_splits, uint32_t page, float scale)
{
    using namespace sgb;
    if (!q || !k_quants || !k_scales || !v_quants || !v_scales || !page_table || !out)
        return set_last_error(3, "decode_noalloc: NULL pointer argument");
    if (device < 0 || device >= 64) return set_last_error(1, "decode_noalloc: device index out of range");
    if (n_kv_heads == 0 || (n_kv_heads & 1)) return set_last_error(3, "decode_noalloc: n_kv_heads must be even and > 0");
    if (m_q == 0 || m_q > 4) return set_last_error(3, "decode_noalloc: m_q must be 1..4");
    if (kv_len == 0 || n_splits == 0) return set_last_error(3, "decode_noalloc: kv_len and n_splits must be > 0");
    if (page == 0 || page % STAGE_TOK) return set_last_error(3, "decode_noalloc: page must be a multiple of 64 tokens");
    const uint64_t part_rows = (uint64_t)m_q * n_kv_heads * G * n_splits;
    if (part_rows > NOALLOC_MAX_PART_ROWS) {
        char buf[200];
        snprintf(buf, sizeof buf,
                 "decode_noalloc: m_q * q_heads * n_splits = %llu partial rows, the static scratch holds at most %u "
                 "(e.g. 32 q heads x 64 splits); use the sgb_dispatch path with a caller-sized buffer instead",
                 (unsigned long long)part_rows, NOALLOC_MAX_PART_ROWS);
        return set_last_error(3, buf);
    }
    if (pool_rows == 0 || pool_rows % page) return set_last_error(3, "decode_noalloc: pool_rows must be whole pages");
    if ((uint64_t)table_len * page < kv_len) return set_last_error(3, "decode_noalloc: page table shorter than kv_len");
    for (const void* p : {k_quants, k_scales, v_quants, v_scales})
        if (reinterpret_cast<uintptr_t>(p) & 15) return set_last_error(3, "decode_noalloc: K/V pools must be 16-byte aligned");

    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return set_last_error(4, std::string("decode_noalloc: selecting the device: ") + cudaGetErrorString(e));
    struct Restore {
        int prev, dev;
        ~Restore()
        {
            if (prev != dev) cudaSetDevice(prev);
        }
    } restore{prev, device};

    // Set-up on the first call per device, with that device current: resolve the device address of
    // the static array and raise the kernel's shared-memory limit.  Neither allocates.
    if (!g_noalloc_ready[device]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return set_last_error(4, std::string("decode_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        e = cudaFuncSetAttribute(decode_paged_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(sizeof(DecodeSmem<4>) + 1024));
        if (e != cudaSuccess)
            return set_last_error(4, std::string("decode_noalloc: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
        g_noalloc_dev_ptr[device] = ptr;
        g_noalloc_ready[device] = true;
    }
    float* scratch = static_cast<float*>(g_noalloc_dev_ptr[device]);
    const uint32_t* step = reinterpret_cast<const uint32_t*>(scratch + NOALLOC_STEP_AT);

    std::string err;
    uint64_t launches = 0;
    LaunchArgs a{(cudaStream_t)stream, nullptr, nullptr, {n_kv_heads, n_splits, m_q}, status, 0, device, &err, &launches};
    const size_t row_bytes = (size_t)n_kv_heads * HD;
    CUtensorMap tm[4];
    const void* quants[2] = {k_quants, v_quants};
    const void* scales[2] = {k_scales, v_scales};
    for (int i = 0; i < 2; i++) {
        const uint64_t qd[3] = {HD, n_kv_heads, pool_rows};
        const uint64_t qs[2] = {HD, row_bytes};
        const uint32_t qb[3] = {HD, 1, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i], 0, 3, const_cast<void*>(quants[i]), qd, qs, qb, 3)) return set_last_error(r, err);
        const uint64_t sd[2] = {(uint64_t)n_kv_heads * 4, pool_rows};
        const uint64_t ss[1] = {(uint64_t)n_kv_heads * 8};
        const uint32_t sb[2] = {8, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i + 1], 1, 2, const_cast<void*>(scales[i]), sd, ss, sb, 0)) return set_last_error(r, err);
    }
    cudaStream_t s = (cudaStream_t)stream;
    noalloc_step_kernel<<<1, 1, 0, s>>>(kv_len);
    decode_paged_kernel<4, 2><<<dim3(n_kv_heads, n_splits), THREADS, sizeof(DecodeSmem<4>) + 1024, s>>>(
        tm[0], tm[1], tm[2], tm[3], (const __half*)q, page_table, table_len, page, (uint32_t)(pool_rows / page), scratch, step,
        n_splits, scale, m_q, status);
    noalloc_reduce_kernel<<<m_q * n_kv_heads * G, HD, 0, s>>>(out, n_splits);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_last_error(4, std::string("decode_noalloc: launch: ") + cudaGetErrorString(e));
    return 0;
}
