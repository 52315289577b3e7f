// Split-K decode / speculative-verify attention over the paged Q8_0 KV cache, head_dim 128.
//
// Semantics: attn_decode_global_q8k (crates/sg-gpu/shaders/attn_decode_global_q8k.wgsl:18-112)
// extended with Q8_0 V, a page table and up to 4 query tokens.  Grid meaning, split ranges
// (chunk = ceil(kv_len / n_splits), l.52-54), the -3e38 sentinel for empty splits (l.68) and the
// partials layout part[(row * n_splits + split) * 130] = acc[128], m, l (l.101-111) are the
// reference's; row = i * H + qh for query token i.
//
// Design (HBM-bound: 17/16 byte per K/V element is all that has to move):
//   * a CTA is four warps = (4 / SUB adjacent kv heads) x (SUB sub-splits of one split); the
//     sub-splits of a head take its 16-token stages round-robin and are merged in fixed order at
//     the end, so the grid fills the SMs in one wave whatever n_splits the caller chose (the
//     partials keep the reference's [row][split][130] layout).  Every warp runs its own
//     pipeline: lane 0 issues the TMA loads of its head's 16-token stages (K quants, V quants, and
//     the 16-byte scale pairs of its head and its neighbour) NSTAGES ahead, through the page
//     table, into the warp's private ring of shared-memory stages; the only synchronisation is the
//     warp's own "full" mbarrier per stage -- no producer warp, no cross-warp barrier;
//   * a warp turns the int8 bytes of its head into exact f16 integers straight out of
//     shared memory (ldmatrix, plain for K and transposed for V, then one byte permute per pair:
//     0x6400 | (q ^ 0x80) = q + 1152) and feeds mma.sync m16n8k16 with the 16 tokens (QK^T) or 16
//     dims (PV) as the M side and the <= 8 query rows as N, so no accumulator row is dead; the
//     tile is far below the 64-row minimum of tcgen05, so the warp-level MMA is the right tool;
//   * the per-block scales never touch the int8 data: QK^T is accumulated per 32-wide block and
//     multiplied by f32(scale) afterwards (sum_b s_b * sum_d q_d k_d == sum_d q_d (s_b k_d), i.e.
//     the reference's exact product f32(scale)*f32(q), no f16 re-rounding); for PV the scale is
//     folded into P.  The +1152 offsets are removed exactly: the QK accumulator starts at
//     -1152 * sum(q) and PV subtracts 1152 * sum(P') gathered by one extra MMA against ones;
//   * online softmax in registers (base 2, row max by warp shuffles over the 4 lanes of a row,
//     rescale only when the max grows by more than 2^8).  A head's tokens are walked by one warp
//     in order, so the partials need no cross-warp merge and reruns are bit-identical.
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include <mutex>
#include <string>

#include "attn_merge.cuh"
#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int HD = 128;
constexpr int G = 2;                     // query heads per kv head
constexpr int STAGE_TOK = 16;            // tokens per pipeline stage = one MMA tile per warp
constexpr uint32_t HEAD_TILE = STAGE_TOK * 128;  // one head's quants of a stage: [16 tokens][128 B]
constexpr uint32_t MAGIC = 0x64646464u;  // high byte of f16 1024.0
constexpr float OFFSET = 1152.0f;        // 1024 + 128
constexpr float RESCALE_T = 8.0f;        // lazy-rescale threshold, log2 units

constexpr int WPC = 4;                   // warps (kv heads) per CTA
constexpr uint32_t SCALE_TILE = STAGE_TOK * 16;  // [16 tokens][2 heads][4 f16]
constexpr uint32_t STAGE_BYTES = 2 * HEAD_TILE + 2 * SCALE_TILE;

template <int NSTAGES>
struct __align__(1024) DecodeSmem {
    uint8_t kq[WPC][NSTAGES][HEAD_TILE];   // 128-byte swizzled by TMA
    uint8_t vq[WPC][NSTAGES][HEAD_TILE];
    uint8_t ks[WPC][NSTAGES][SCALE_TILE];
    uint8_t vs[WPC][NSTAGES][SCALE_TILE];
    uint64_t full[WPC][NSTAGES];
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Transpose an 8x8 matrix of 16-bit elements held one row-pair per lane (the mma C/B layouts).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint2 lds_u2(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b)
{
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Reductions over the 8 lanes that share t4 (lane bits 2..4): the tokens of a tile.
__device__ __forceinline__ float tok_max(float v)
{
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float tok_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v + __shfl_xor_sync(0xffffffffu, v, 16);
}
__device__ __forceinline__ float quad_sum(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int NSTAGES, int MIN_CTAS, int SUB>
__global__ void __launch_bounds__(WPC * 32, MIN_CTAS)
    decode_paged_kernel(const __grid_constant__ CUtensorMap tm_kq, const __grid_constant__ CUtensorMap tm_ks,
                        const __grid_constant__ CUtensorMap tm_vq, const __grid_constant__ CUtensorMap tm_vs,
                        const __half* __restrict__ q, const uint32_t* __restrict__ page_table, uint32_t table_len, uint32_t page,
                        uint32_t pool_pages, float* __restrict__ part, const uint32_t* __restrict__ step, uint32_t n_kv,
                        uint32_t n_splits, float scale, uint32_t m_q, uint32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    using Smem = DecodeSmem<NSTAGES>;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    static_assert(NSTAGES * HEAD_TILE >= 8 * (HD + 2) * 4, "a warp's K ring doubles as its merge buffer");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int HEADS_PER_CTA = WPC / SUB;
    const int kvh = blockIdx.x * HEADS_PER_CTA + warp / SUB, sub = warp % SUB, split = blockIdx.y;
    const int n_q = (int)n_kv * G;
    const bool active = kvh < (int)n_kv;  // idle warps of the last CTA when n_kv * SUB is not a multiple of 4
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t rows = m_q * G;

    if (lane == 0) {
        tma_prefetch_desc(&tm_kq);
        tma_prefetch_desc(&tm_vq);
        for (int i = 0; i < NSTAGES; i++) mbar_init(&sm.full[warp][i], 1);
        mbar_fence_init();
    }
    pdl_wait();  // everything below reads what earlier kernels of the stream wrote (step words, q, the appended rows)
    pdl_launch_dependents();
    const uint32_t kv_len = __ldg(step + STEP_KV_LEN_GLOBAL);
    const uint32_t chunk = (kv_len + n_splits - 1) / n_splits;
    const uint32_t t_begin = min((uint32_t)split * chunk, kv_len);
    const uint32_t t_end = min(t_begin + chunk, kv_len);
    const uint32_t s_begin = t_begin / STAGE_TOK + sub;  // this warp's first stage; it then strides by SUB
    const uint32_t n_stages = t_begin < t_end ? (t_end + STAGE_TOK - 1) / STAGE_TOK - t_begin / STAGE_TOK : 0;
    const uint32_t n_iter = active && n_stages > (uint32_t)sub ? (n_stages - sub + SUB - 1) / SUB : 0;
    __syncwarp();

    const uint32_t page_shift = 31 - __clz(page);
    // Physical page of the stage with index `stage` (tokens 16*stage ..), checked, never followed blindly.
    auto lookup = [&](uint32_t stage) -> uint32_t {
        const uint32_t lp = (stage * STAGE_TOK) >> page_shift;  // page is a power of two (checked on the host)
        uint32_t pp = 0;
        if (lp < table_len) {
            pp = __ldg(page_table + lp);
        } else {
            report_error(status, DEV_ERR_BOUNDS, 302, lp, table_len);
        }
        if (pp >= pool_pages) {
            report_error(status, DEV_ERR_BOUNDS, 303, pp, pool_pages);
            pp = 0;
        }
        return pp;
    };
    // Lanes 0..3 start the four TMA copies of iteration `it` into slot it % NSTAGES with ONE instruction:
    // lane 0 = K quants, 1 = K scales, 2 = V quants, 3 = V scales (all four are 3-D copies).
    const CUtensorMap* my_map = lane == 0 ? &tm_kq : lane == 1 ? &tm_ks : lane == 2 ? &tm_vq : &tm_vs;
    const uint32_t my_dst0 = lane == 0 ? smem_u32(sm.kq[warp][0]) : lane == 1 ? smem_u32(sm.ks[warp][0])
                           : lane == 2 ? smem_u32(sm.vq[warp][0]) : smem_u32(sm.vs[warp][0]);
    const uint32_t my_stride = (lane & 1) ? SCALE_TILE : HEAD_TILE;
    const int my_c1 = (lane & 1) ? (kvh >> 1) : kvh;
    const uint32_t bar0 = smem_u32(&sm.full[warp][0]);
    auto issue = [&](uint32_t it, uint32_t pp) {
        const uint32_t st = it % NSTAGES;
        const uint32_t tok0 = (s_begin + it * SUB) * STAGE_TOK;
        const int row = (int)((pp << page_shift) + (tok0 & (page - 1)));
        const uint32_t bar = bar0 + st * 8;
        if (lane == 0) {
            fence_proxy_async_smem();  // the slot's previous contents were read through the generic proxy
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
        }
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(my_dst0 + st * my_stride), "l"(reinterpret_cast<uint64_t>(my_map)), "r"(bar), "r"(0), "r"(my_c1), "r"(row)
            : "memory");
    };
    // Start the pipeline before anything else: lanes 0..NSTAGES-1 fetch the first page entries side
    // by side (one memory latency, not NSTAGES), lane 0 issues; the Q loads below overlap the copies.
    {
        const uint32_t n_pre = min(n_iter, (uint32_t)NSTAGES);
        uint32_t my_pp = 0;
        if ((uint32_t)lane < n_pre) my_pp = lookup(s_begin + lane * SUB);
        for (uint32_t it = 0; it < n_pre; ++it) {
            const uint32_t pp = __shfl_sync(0xffffffffu, my_pp, it);
            if (lane < 4) issue(it, pp);
        }
    }
    // The page of the next stage to be issued is looked up one iteration early, so the load's
    // latency is covered by a tile of work.
    uint32_t next_pp = 0;
    if (n_iter > (uint32_t)NSTAGES && lane < 4) next_pp = lookup(s_begin + NSTAGES * SUB);

    // MMA roles.  QK^T: A = K (16 tokens x 16 dims of chunk c), B = Q^T (16 dims x 8 query rows).
    //            PV  : A = V^T (16 dims of chunk c x 16 tokens), B = P'^T (16 tokens x 8 query rows).
    // A lane therefore supplies Q for query row g (B operand) and owns the accumulator columns of
    // query rows 2*t4 and 2*t4 + 1 (C operand).
    //
    // Q as B fragments: ldmatrix hands lane t4 the bytes 4*t4 .. 4*t4+3 of every 16-byte chunk of a K
    // row, so k-step c contracts dims 16c + 4*t4 + {0,1 | 2,3}.
    uint32_t qb[8][2];
    float cinit[4][2];  // -1152 * (sum of q over block b) for query rows 2*t4 + e
    {
        const bool q_live = active && (uint32_t)g < rows;
        const __half* qrow = q + ((size_t)(g / G) * n_q + kvh * G + g % G) * HD;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            float sum = 0.0f;
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const int c = 2 * b + cc;
                uint2 w = make_uint2(0u, 0u);
                if (q_live) w = __ldg(reinterpret_cast<const uint2*>(qrow + 16 * c + 4 * t4));
                qb[c][0] = w.x;
                qb[c][1] = w.y;
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
                sum += (f0.x + f0.y) + (f1.x + f1.y);
            }
            sum = -OFFSET * quad_sum(sum);  // now the block sum of query row g, in all 4 lanes of the quad
            cinit[b][0] = __shfl_sync(0xffffffffu, sum, (2 * t4) * 4);
            cinit[b][1] = __shfl_sync(0xffffffffu, sum, (2 * t4 + 1) * 4);
        }
    }
    // Keys query row 2*t4 + e may see: [t_begin, hi_row[e]], hi = min(t_end - 1, kv_len - m_q + token index).
    int hi_row[2];
#pragma unroll
    for (int e = 0; e < 2; e++) hi_row[e] = min((int)t_end - 1, (int)kv_len - (int)m_q + (2 * t4 + e) / G);
    const int hi_all = min((int)t_end - 1, (int)kv_len - (int)m_q);  // visible to every row

    // Per-lane shared-memory offsets (bytes) inside a head tile [16 tokens][128 B, swizzled].  For both
    // K (plain) and V (transposed) one ldmatrix.x4 fetches block b: lane l addresses row (l & 7) of
    // matrix (l >> 3) = (token half (l >> 3) & 1, 16-byte chunk 2b + (l >> 4)).
    const uint32_t lrow = lane & 7, lmat = lane >> 3;
    uint32_t off[4];
#pragma unroll
    for (int b = 0; b < 4; b++) off[b] = (8 * (lmat & 1) + lrow) * 128 + (((2 * b + (lmat >> 1)) ^ lrow) << 4);
    // scales: [token][2 heads][4 f16].  K side: tokens g and g + 8; V side: tokens 2*t4 + e and 8 + 2*t4 + e.
    const uint32_t ksc_off = g * 16 + (kvh & 1) * 8;
    const uint32_t vsc_off = (2 * t4) * 16 + (kvh & 1) * 8;

    const float scale2 = scale * 1.4426950408889634f;
    float m_run[2] = {NEG_SENTINEL, NEG_SENTINEL}, l_part[2] = {0.0f, 0.0f};
    float o[8][4];     // o[c]: dims 16c + 2g (c0, c1) and 16c + 2g + 1 (c2, c3) x query rows 2*t4 (c0, c2), 2*t4 + 1 (c1, c3)
    float osum[4][4];  // per block: sum over tokens of P'_b, same column layout
#pragma unroll
    for (int c = 0; c < 8; c++) o[c][0] = o[c][1] = o[c][2] = o[c][3] = 0.0f;
#pragma unroll
    for (int b = 0; b < 4; b++) osum[b][0] = osum[b][1] = osum[b][2] = osum[b][3] = 0.0f;
    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};

    bool failed = false;
    for (uint32_t it = 0; it < n_iter; ++it) {
        const int st = it % NSTAGES;
        mbar_wait(&sm.full[warp][st], (it / NSTAGES) & 1, status, 305, failed);
        const int tok0 = (int)((s_begin + it * SUB) * STAGE_TOK);
        const uint32_t kq_base = smem_u32(sm.kq[warp][st]), vq_base = smem_u32(sm.vq[warp][st]);

        // ---- S = K Q^T per 32-wide block, then the block scales: s[th][e] = score of token g + 8*th
        //      against query row 2*t4 + e -----------------------------------------------------------
        float s[2][2];
        {
            const uint2 sa = lds_u2(smem_u32(sm.ks[warp][st]) + ksc_off);        // scales of token g
            const uint2 sb = lds_u2(smem_u32(sm.ks[warp][st]) + ksc_off + 128);  // scales of token g + 8
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(&sa.x));
            const float2 a23 = __half22float2(*reinterpret_cast<const __half2*>(&sa.y));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&sb.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&sb.y));
            const float ka[4] = {a01.x, a01.y, a23.x, a23.y}, kb[4] = {b01.x, b01.y, b23.x, b23.y};
            s[0][0] = s[0][1] = s[1][0] = s[1][1] = 0.0f;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                uint32_t x[4];  // (token half 0, chunk 2b), (1, 2b), (0, 2b+1), (1, 2b+1): bytes 4*t4.. of token g (+8)
                ldsm_x4(kq_base + off[b], x);
                float acc[4] = {cinit[b][0], cinit[b][1], cinit[b][0], cinit[b][1]};
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
                    const uint32_t x0 = x[2 * cc] ^ 0x80808080u, x1 = x[2 * cc + 1] ^ 0x80808080u;
                    const uint32_t a[4] = {__byte_perm(x0, MAGIC, 0x4140), __byte_perm(x1, MAGIC, 0x4140),
                                           __byte_perm(x0, MAGIC, 0x4342), __byte_perm(x1, MAGIC, 0x4342)};
                    mma16816(acc, a, qb[2 * b + cc][0], qb[2 * b + cc][1]);
                }
                s[0][0] = fmaf(ka[b], acc[0], s[0][0]);
                s[0][1] = fmaf(ka[b], acc[1], s[0][1]);
                s[1][0] = fmaf(kb[b], acc[2], s[1][0]);
                s[1][1] = fmaf(kb[b], acc[3], s[1][1]);
            }
        }
#pragma unroll
        for (int th = 0; th < 2; th++) {
            s[th][0] *= scale2;
            s[th][1] *= scale2;
        }
        // Masks only on the stages that straddle the split's ends or the causal edge of the draft.
        if (tok0 < (int)t_begin || tok0 + STAGE_TOK - 1 > hi_all) {
#pragma unroll
            for (int th = 0; th < 2; th++) {
                const int T = tok0 + g + 8 * th;
#pragma unroll
                for (int e = 0; e < 2; e++)
                    if (T < (int)t_begin || T > hi_row[e]) s[th][e] = -INFINITY;
            }
        }
        const float mx0 = tok_max(fmaxf(s[0][0], s[1][0])), mx1 = tok_max(fmaxf(s[0][1], s[1][1]));
        const bool grow0 = mx0 > m_run[0] + RESCALE_T, grow1 = mx1 > m_run[1] + RESCALE_T;
        if (__any_sync(0xffffffffu, grow0 || grow1)) {
            const float n0 = grow0 ? mx0 : m_run[0], n1 = grow1 ? mx1 : m_run[1];
            const float c0 = ex2(m_run[0] - n0), c1 = ex2(m_run[1] - n1);
            m_run[0] = n0;
            m_run[1] = n1;
            l_part[0] *= c0;
            l_part[1] *= c1;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                o[c][0] *= c0;
                o[c][1] *= c1;
                o[c][2] *= c0;
                o[c][3] *= c1;
            }
#pragma unroll
            for (int b = 0; b < 4; b++) {
                osum[b][0] *= c0;
                osum[b][1] *= c1;
                osum[b][2] *= c0;
                osum[b][3] *= c1;
            }
        }
        const float p00 = ex2(s[0][0] - m_run[0]), p01 = ex2(s[0][1] - m_run[1]);
        const float p10 = ex2(s[1][0] - m_run[0]), p11 = ex2(s[1][1] - m_run[1]);
        l_part[0] += p00 + p10;
        l_part[1] += p01 + p11;

        // ---- P (tokens x query rows) -> P^T fragments: lane (g, t4) gets query row g, tokens 2*t4, 2*t4+1
        //      (and 8 + those); then P'_b = P * (V scale of block b), and O^T += V^T P'^T ----------------
        const uint32_t pt0 = movmatrix_trans(pack_half2(p00, p01));
        const uint32_t pt1 = movmatrix_trans(pack_half2(p10, p11));
        const uint32_t vs_base = smem_u32(sm.vs[warp][st]) + vsc_off;
        uint2 va = lds_u2(vs_base), vb = lds_u2(vs_base + 16);              // tokens 2*t4, 2*t4+1
        uint2 vc = lds_u2(vs_base + 8 * 16), vd = lds_u2(vs_base + 9 * 16);  // tokens 8+2*t4, 9+2*t4
        if (tok0 + STAGE_TOK > (int)kv_len) {
            // Rows past the end of the sequence hold whatever was there before; their p is 0, but 0 times a
            // stale scale that happens to be inf or NaN would not be.
            const uint2 zero = make_uint2(0u, 0u);
            if (tok0 + 2 * t4 >= (int)kv_len) va = zero;
            if (tok0 + 2 * t4 + 1 >= (int)kv_len) vb = zero;
            if (tok0 + 8 + 2 * t4 >= (int)kv_len) vc = zero;
            if (tok0 + 9 + 2 * t4 >= (int)kv_len) vd = zero;
        }
#pragma unroll
        for (int b = 0; b < 4; b++) {
            // (scale_b of token A, scale_b of token B) as a half2, times (p_A, p_B)
            const uint32_t sel = (b & 1) ? 0x7632u : 0x5410u;
            const uint32_t pb0 = hmul2_u32(pt0, __byte_perm(b < 2 ? va.x : va.y, b < 2 ? vb.x : vb.y, sel));
            const uint32_t pb1 = hmul2_u32(pt1, __byte_perm(b < 2 ? vc.x : vc.y, b < 2 ? vd.x : vd.y, sel));
            uint32_t y[4];  // transposed: bytes V[8th + 2*t4 (+1)][16c + 2g (+1)] for (th, c) = (0,2b),(1,2b),(0,2b+1),(1,2b+1)
            ldsm_x4_trans(vq_base + off[b], y);
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const uint32_t y0 = y[2 * cc] ^ 0x80808080u, y1 = y[2 * cc + 1] ^ 0x80808080u;
                const uint32_t a[4] = {__byte_perm(y0, MAGIC, 0x4240), __byte_perm(y0, MAGIC, 0x4341),
                                       __byte_perm(y1, MAGIC, 0x4240), __byte_perm(y1, MAGIC, 0x4341)};
                mma16816(o[2 * b + cc], a, pb0, pb1);
            }
            mma16816(osum[b], ones, pb0, pb1);
        }

        // Refill this slot for iteration it + NSTAGES; every lane is done reading it.
        __syncwarp();
        if (lane < 4 && it + NSTAGES < n_iter) {
            issue(it + NSTAGES, next_pp);
            if (it + NSTAGES + 1 < n_iter) next_pp = lookup(s_begin + (it + NSTAGES + 1) * SUB);
        }
    }

    // ---- remove the +1152 offsets, total the denominators --------------------------------------------
#pragma unroll
    for (int c = 0; c < 8; c++) {
#pragma unroll
        for (int i = 0; i < 4; i++) o[c][i] -= OFFSET * osum[c >> 1][i];
    }
    float l_row[2] = {tok_sum(l_part[0]), tok_sum(l_part[1])};

    // ---- merge the SUB sub-splits of a head in fixed order (sub 0 <- 1 <- 2 <- 3) ----------------------
    // A warp's K ring is free by now (all its copies were consumed) and holds [8 rows][130] floats.
    if (SUB > 1) {
        float* mine = reinterpret_cast<float*>(sm.kq[warp][0]);
        if (sub != 0) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                float* dst = mine + (2 * t4 + e) * (HD + 2);
#pragma unroll
                for (int c = 0; c < 8; c++) *reinterpret_cast<float2*>(dst + 16 * c + 2 * g) = make_float2(o[c][e], o[c][2 + e]);
                if (g == 0) {
                    dst[HD] = m_run[e];
                    dst[HD + 1] = l_row[e];
                }
            }
        }
        __syncthreads();
        if (sub == 0) {
#pragma unroll
            for (int u = 1; u < SUB; u++) {
                const float* other = reinterpret_cast<const float*>(sm.kq[warp + u][0]);
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float* src = other + (2 * t4 + e) * (HD + 2);
                    const float mo = src[HD], lo = src[HD + 1];
                    const float mn = fmaxf(m_run[e], mo);
                    const float fa = ex2(m_run[e] - mn), fb = ex2(mo - mn);
                    m_run[e] = mn;
                    l_row[e] = l_row[e] * fa + lo * fb;
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const float2 v = *reinterpret_cast<const float2*>(src + 16 * c + 2 * g);
                        o[c][e] = o[c][e] * fa + v.x * fb;
                        o[c][2 + e] = o[c][2 + e] * fa + v.y * fb;
                    }
                }
            }
        }
    }

    // ---- the split's partial, straight from registers ------------------------------------------------
    if (active && sub == 0) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t r = 2 * t4 + e;  // query row = token index * G + head within the group
            if (r < rows) {
                float* dst = part + (((size_t)(r / G) * n_q + kvh * G + r % G) * n_splits + split) * (HD + 2);
                // dims 16c + 2g and 16c + 2g + 1; rows are 520 bytes, so 8-byte aligned stores
#pragma unroll
                for (int c = 0; c < 8; c++) *reinterpret_cast<float2*>(dst + 16 * c + 2 * g) = make_float2(o[c][e], o[c][2 + e]);
                if (g == 0) {
                    dst[HD] = m_run[e] == NEG_SENTINEL ? NEG_SENTINEL : m_run[e] * 0.6931471805599453f;  // back to natural log
                    dst[HD + 1] = l_row[e];
                }
            }
        }
    }
}

struct PushDecodePaged {
    uint32_t n_splits;
    float scale;
    uint32_t page;
};

// Tensor maps of the four pools: quants as [row][kv head][128] u8 with a (128, 1, 16) box and the
// 128-byte swizzle, scales as [row][kv heads * 4] f16 with a (hpc * 4, 16) box.
int encode_pool_maps(const LaunchArgs& a, CUtensorMap (&tm)[4], const void* const (&quants)[2], const void* const (&scales)[2],
                     uint32_t n_kv, uint64_t pool_rows)
{
    for (int i = 0; i < 2; i++) {
        const uint64_t qd[3] = {HD, n_kv, pool_rows};
        const uint64_t qs[2] = {HD, (uint64_t)n_kv * HD};
        const uint32_t qb[3] = {HD, 1, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i], 0, 3, const_cast<void*>(quants[i]), qd, qs, qb, 3)) return r;
        const uint64_t sd[3] = {8, (uint64_t)n_kv / 2, pool_rows};
        const uint64_t ss[2] = {16, (uint64_t)n_kv * 8};
        const uint32_t sb[3] = {8, 1, STAGE_TOK};
        if (int r = encode_tensor_map(a, &tm[2 * i + 1], 1, 3, const_cast<void*>(scales[i]), sd, ss, sb, 0)) return r;
    }
    return 0;
}

template <int NSTAGES, int MIN_CTAS, int SUB>
cudaError_t launch_decode_variant(cudaStream_t stream, int device, const CUtensorMap (&tm)[4], const __half* q,
                                  const uint32_t* page_table, uint32_t table_len, uint32_t page, uint32_t pool_pages, float* part,
                                  const uint32_t* step, uint32_t n_kv, uint32_t n_splits, float scale, uint32_t m_q, uint32_t* status)
{
    using Smem = DecodeSmem<NSTAGES>;
    const size_t smem = sizeof(Smem) + 1024;
    static std::mutex attr_mutex;
    static bool attr_set[64] = {};
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        if (device >= 0 && device < 64 && !attr_set[device]) {
            cudaError_t e = cudaFuncSetAttribute(decode_paged_kernel<NSTAGES, MIN_CTAS, SUB>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            attr_set[device] = true;
        }
    }
    const uint32_t ctas_x = (n_kv * SUB + WPC - 1) / WPC;
    return launch_dependent(decode_paged_kernel<NSTAGES, MIN_CTAS, SUB>, dim3(ctas_x, n_splits), dim3(WPC * 32), smem, stream, tm[0],
                            tm[1], tm[2], tm[3], q, page_table, table_len, page, pool_pages, part, step, n_kv, n_splits, scale, m_q, status);
}

// Shape of the launch.  Three 4.5 KB stages per warp = 54 KB per CTA and 128 registers per thread let
// four CTAs = 16 warps live on an SM.  The number of sub-splits per (kv head, split) is the largest
// of 4, 2, 1 for which all warps still fit on the GPU at once (one wave): extra waves cost more
// than the parallelism buys.  SGB_DECODE_SUB=1|2|4 overrides the choice (tuning aid; results agree
// within rounding, each choice is bit-reproducible).
cudaError_t launch_decode(cudaStream_t stream, int device, int sm_count, const CUtensorMap (&tm)[4], const __half* q,
                          const uint32_t* page_table, uint32_t table_len, uint32_t page, uint32_t pool_pages, float* part,
                          const uint32_t* step, uint32_t n_kv, uint32_t n_splits, float scale, uint32_t m_q, uint32_t* status)
{
    static const int forced = [] {
        const char* e = getenv("SGB_DECODE_SUB");
        return e ? atoi(e) : 0;
    }();
    const uint64_t slots = (uint64_t)(sm_count > 0 ? sm_count : 148) * 16;
    const uint64_t tasks = (uint64_t)n_kv * n_splits;
    int sub = tasks * 4 <= slots ? 4 : tasks * 2 <= slots ? 2 : 1;
    if (forced == 1 || forced == 2 || forced == 4) sub = forced;
#define SGB_DECODE_ARGS stream, device, tm, q, page_table, table_len, page, pool_pages, part, step, n_kv, n_splits, scale, m_q, status
    if (sub == 4) return launch_decode_variant<3, 4, 4>(SGB_DECODE_ARGS);
    if (sub == 2) return launch_decode_variant<3, 4, 2>(SGB_DECODE_ARGS);
    return launch_decode_variant<3, 4, 1>(SGB_DECODE_ARGS);
#undef SGB_DECODE_ARGS
}

}  // namespace

// attn_decode_paged_q8kv_d128 / attn_verify_paged_q8kv_d128.
// bindings: q f16 [m_q x H x 128], k_quants i8, k_scales f16, v_quants i8, v_scales f16,
//           page_table u32, part f32 [m_q*H x n_splits x 130], step.
// push {n_splits u32, scale f32, page u32}.  grid [n_kv_heads, n_splits, m_q (0 or 1 = decode)].
int launch_decode_paged_q8kv_d128(const LaunchArgs& a)
{
    const PushDecodePaged p = *(const PushDecodePaged*)a.push;
    const uint32_t n_kv = a.groups[0];
    const uint32_t m_q = a.groups[2] ? a.groups[2] : 1;
    if (n_kv == 0 || (n_kv & 1)) return fail_validation(a, "decode_paged: groups[0] (kv heads) must be even and > 0");
    if (p.n_splits == 0 || a.groups[1] != p.n_splits)
        return fail_validation(a, "decode_paged: groups[1] must equal push.n_splits (> 0)");
    if (m_q > 4) return fail_validation(a, "decode_paged: at most 4 query tokens");
    if (p.page < (uint32_t)STAGE_TOK || (p.page & (p.page - 1)))
        return fail_validation(a, "decode_paged: page must be a power of two, at least 16 tokens");
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
    const void* const quants[2] = {a.b[1].ptr, a.b[3].ptr};
    const void* const scales[2] = {a.b[2].ptr, a.b[4].ptr};
    if (int r = encode_pool_maps(a, tm, quants, scales, n_kv, pool_rows)) return r;
    const cudaError_t e = launch_decode(a.stream, a.device, a.sm_count, tm, (const __half*)a.b[0].ptr, (const uint32_t*)a.b[5].ptr,
                                        (uint32_t)(a.b[5].bytes / 4), p.page, (uint32_t)(pool_rows / p.page), (float*)a.b[6].ptr,
                                        (const uint32_t*)a.b[7].ptr, n_kv, p.n_splits, p.scale, m_q, a.status);
    ++*a.launches;
    return check_cuda(a, e, "attn_decode_paged_q8kv_d128");
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
std::mutex g_noalloc_mutex;  // the per-device set-up may be reached from several host threads

__global__ void noalloc_step_kernel(uint32_t kv_len)
{
    uint32_t* step = reinterpret_cast<uint32_t*>(g_noalloc_scratch + NOALLOC_STEP_AT);
    step[STEP_POS] = 0;
    step[STEP_KV_LEN_SLIDING] = 0;
    step[STEP_KV_LEN_GLOBAL] = kv_len;
    step[STEP_Q0] = 0;
}

// Combine of the splits: the shared statement of attn_reduce.wgsl:29-56 (merge_splits_running, the arithmetic
// of attn_reduce_f32_d128, so both decode entries give the same bits), reading the partials straight from the
// static array.  One block per query row, two dims per thread.
__global__ void __launch_bounds__(HD / 2) noalloc_reduce_kernel(float* __restrict__ out, uint32_t n_splits)
{
    const size_t row = blockIdx.x;
    const int d0 = 2 * threadIdx.x;
    float acc[2];
    const MergeState st = merge_splits_running<HD, 2, 3>(g_noalloc_scratch + row * n_splits * (HD + 2), HD + 2, n_splits, d0, acc);
    *reinterpret_cast<float2*>(out + row * HD + d0) = make_float2(acc[0] / st.l, acc[1] / st.l);
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
    if (kv_len < m_q) return set_last_error(3, "decode_noalloc: kv_len counts the m_q query tokens, so it cannot be smaller than m_q");
    if (page < (uint32_t)STAGE_TOK || (page & (page - 1)))
        return set_last_error(3, "decode_noalloc: page must be a power of two, at least 16 tokens");
    const uint64_t part_rows = (uint64_t)m_q * n_kv_heads * G * n_splits;
    if (part_rows > NOALLOC_MAX_PART_ROWS) {
        char buf[320];
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
    // the static array (the decode launcher raises its kernel's shared-memory limit on its own first
    // use per device).  Neither call allocates by itself, but this is where the CUDA runtime loads the
    // module that holds the array on this device (module loading is lazy), and that is when the driver
    // sets the array's 1.04 MB aside: the first call per device must come while that much is still free.
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ready[device]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return set_last_error(4, std::string("decode_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_noalloc_dev_ptr[device] = ptr;
        g_noalloc_ready[device] = true;
    }
    float* scratch = static_cast<float*>(g_noalloc_dev_ptr[device]);
    const uint32_t* step = reinterpret_cast<const uint32_t*>(scratch + NOALLOC_STEP_AT);

    std::string err;
    uint64_t launches = 0;
    LaunchArgs a{(cudaStream_t)stream, nullptr, nullptr, {n_kv_heads, n_splits, m_q}, status, 0, device, &err, &launches};
    CUtensorMap tm[4];
    const void* const quants[2] = {k_quants, v_quants};
    const void* const scales[2] = {k_scales, v_scales};
    if (int r = encode_pool_maps(a, tm, quants, scales, n_kv_heads, pool_rows)) return set_last_error(r, err);
    cudaStream_t s = (cudaStream_t)stream;
    noalloc_step_kernel<<<1, 1, 0, s>>>(kv_len);
    int sm_count = 0;
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    e = launch_decode(s, device, sm_count, tm, (const __half*)q, page_table, table_len, page, (uint32_t)(pool_rows / page), scratch, step,
                      n_kv_heads, n_splits, scale, m_q, status);
    if (e != cudaSuccess) return set_last_error(4, std::string("decode_noalloc: launch: ") + cudaGetErrorString(e));
    noalloc_reduce_kernel<<<m_q * n_kv_heads * G, HD / 2, 0, s>>>(out, n_splits);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_last_error(4, std::string("decode_noalloc: launch: ") + cudaGetErrorString(e));
    return 0;
}
