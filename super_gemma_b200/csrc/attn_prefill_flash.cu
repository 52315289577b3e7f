// Flash-attention prefill on tcgen05 tensor cores, head_dim 128, GQA 2.
//
// Semantics: single-pass online-softmax flash attention as attn_prefill_global_flash_sp.wgsl:118-188
// (m_new = max over visible s*scale, p = exp(s*scale - m), l += p in f32 BEFORE P = f16(p),
// O = O*corr + P*V, out = O / l), with the banded mask of attn_prefill_sliding.wgsl:53-57 and the
// ring + chunk key sources of attn_prefill_sliding_ring.wgsl:88-140 as variants.  The Q8_0 paged
// entry dequantises to f16(scale*q) first (the value attn_prefill_global_flash_sp_q8.wgsl:104
// builds), then runs the same kernel.  Output is f32.
//
// One CTA = 64 query tokens x the 2 query heads of one kv head = 128 rows of S and O, so both
// heads share every K/V tile (GQA grouping).  Per 64-key tile:
//   TMA (128B swizzle, CTA-local) -> smem K, V                 loader warp
//   S[128x64]  = Q K^T   tcgen05.mma kind::f16, D in TMEM      MMA warp, 8 instructions (K = 16 each)
//   row softmax in registers: thread r owns TMEM lane r (tcgen05.ld 32x32b), base-2 exponent,
//       running max raised only when it grows by > 2^8; masked tiles only at the band edges,
//       tiles wholly outside [qpos+1-window, qpos] are never visited           4 softmax warps
//   P -> back into tensor memory over S as packed f16 pairs (tcgen05.st)
//   O[128x128] += P V    tcgen05.mma with A = P from tensor memory, V as the MN-major B operand straight
//                        from its [key][dim] tile
// S is double-buffered in TMEM and the three roles talk through mbarriers only, so Q K^T of the
// next tile and P V of the previous one run while the softmax warps work.  Two CTAs fit per SM
// (96 KB smem, 256 TMEM columns each).  Every mbarrier wait is bounded; TMEM is always freed.
#include <cmath>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

int run_kv_dequant_paged(const LaunchArgs& a, const BufView& scales, const BufView& quants, const BufView& table,
                         const BufView& dst, const BufView& step, uint32_t row_len, uint32_t page);

namespace {

constexpr int HD = 128;
constexpr int G = 2;
constexpr int BLOCK_TOK = 64;   // query tokens per CTA
constexpr int BLOCK_M = 128;    // rows = tokens x G
constexpr int BLOCK_N = 64;     // keys per tile
constexpr int SOFTMAX_THREADS = 128;
constexpr int MMA_WARP = 4, LOAD_WARP = 5;
constexpr int FLASH_THREADS = 192;
constexpr int KV_STAGES = 2;
constexpr uint32_t HALF_TILE = 64 * 128;           // one [64 rows][128 B] box
constexpr uint32_t Q_BYTES = 2 * 2 * HALF_TILE;    // 2 dim-halves x 128 rows
constexpr uint32_t KV_TILE_BYTES = 2 * HALF_TILE;  // 2 dim-halves x 64 keys
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t TMEM_S = 0;     // S: two buffers of 64 f32 columns
constexpr uint32_t TMEM_O = 128;   // O: 128 f32 columns
constexpr float RESCALE_T = 8.0f;

// 96 KB of tiles + 128 B of barriers.  Two CTAs must fit in the SM's 228 KB next to the 1 KB the
// system reserves per CTA, so the struct is NOT padded to its 1024-byte tile alignment: the dynamic
// shared-memory base is declared 1024-aligned instead (and checked at run time).
struct FlashSmem {
    uint8_t q[2][2 * HALF_TILE];             // [dim half][128 rows x 128 B]
    uint8_t k[KV_STAGES][2][HALF_TILE];      // [stage][dim half][64 keys x 128 B]
    uint8_t v[KV_STAGES][2][HALF_TILE];
    uint64_t full_k[KV_STAGES];              // TMA -> MMA warp
    uint64_t full_v[KV_STAGES];
    uint64_t s_ready[2];                     // MMA commit: S[b] holds Q K^T of a tile
    uint64_t q_bar;
    // p_ready and pv_done are indexed by tile parity like S: a producer can then never be two phases
    // ahead of a consumer that has not polled yet, whatever the relative speed of the roles.
    uint64_t p_ready[2];                     // 128 softmax threads: P(j) is in tensor memory
    uint64_t pv_done[2];                     // MMA commit: O += P V of a tile has completed
    uint32_t tmem_base;
    uint32_t abort;                          // a bounded wait ran out somewhere in the CTA
    uint32_t pad[8];
};
static_assert(sizeof(FlashSmem) == 6 * 2 * HALF_TILE + 128, "tiles + barriers, no padding");
static_assert(2 * (sizeof(FlashSmem) + 1024) <= 228 * 1024, "two CTAs per SM");

struct FlashParams {
    const uint32_t* step;
    float* out;
    float* part_acc;     // pieces > 1: [row][piece][128] unnormalised O
    float* part_ml;      // pieces > 1: [row][piece][2] = running max (base-2 exponent units), sum
    uint32_t* status;
    uint32_t m_tokens;   // query tokens in the chunk
    uint32_t n_kv;
    uint32_t window;     // 0 = none
    uint32_t ring;       // TWO_SRC: ring slots
    float scale;
    uint32_t head_group; // kv heads whose query tiles are interleaved in launch order (divides n_kv)
};

// One 64-key tile: where it comes from and which absolute positions its rows hold.
struct Tile {
    int src;        // 0 = history / linear, 1 = chunk
    int row0;       // TMA row coordinate of key 0 of the tile
    int64_t pos0;   // absolute position of key 0
    int64_t lo, hi; // positions of this source that are real: [lo, hi]
};

// Roles: warps 0-3 = softmax (thread r owns row r of S and O), warp 4 = MMA issue (one thread),
// warp 5 = TMA loads (one thread).  Per tile j the tensor pipe runs, in order, ... PV(j-1) QK(j+1)
// PV(j) QK(j+2) ...: S is double-buffered in TMEM, so QK(j+1) and PV(j-1) execute while the softmax
// warps work on tile j, and the softmax is the only thing on the critical path of a CTA; the second
// CTA on the SM fills the tensor pipe's remaining gaps.
template <bool TWO_SRC>
__global__ void __launch_bounds__(FLASH_THREADS, 2) flash_prefill_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                         const __grid_constant__ CUtensorMap tm_k0,
                                                                         const __grid_constant__ CUtensorMap tm_v0,
                                                                         const __grid_constant__ CUtensorMap tm_k1,
                                                                         const __grid_constant__ CUtensorMap tm_v1,
                                                                         const FlashParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    FlashSmem& sm = *reinterpret_cast<FlashSmem*>(smem_raw);
    if ((smem_u32(smem_raw) & 1023u) != 0u) {  // the swizzled tiles need it; never seen, but never assumed
        if (threadIdx.x == 0) report_error(prm.status, DEV_ERR_BOUNDS, 400, smem_u32(smem_raw), 0);
        return;
    }

    const int tid = threadIdx.x, warp = tid >> 5;
    // Launch order (blockIdx.x, then pieces): groups of `head_group` kv heads one after the other; inside a group the latest
    // query tile (the one with the most keys) of every head first, then the one before it, and so on.  The CTAs that run
    // together then read the K/V of one group, which the launcher sizes to stay in L2, and within the group the short
    // CTAs fill the end.
    const int n_qtiles = (int)((prm.m_tokens + BLOCK_TOK - 1) / BLOCK_TOK);
    const uint32_t per_group = prm.head_group * (uint32_t)n_qtiles;
    const uint32_t in_group = blockIdx.x % per_group;
    const int qt = n_qtiles - 1 - (int)(in_group / prm.head_group);
    const int kvh = (int)((blockIdx.x / per_group) * prm.head_group + in_group % prm.head_group);
    const uint32_t m0 = (uint32_t)qt * BLOCK_TOK;
    const int64_t q0 = prm.step[STEP_Q0];
    const uint32_t tok_in_tile = min((uint32_t)BLOCK_TOK, prm.m_tokens - m0);

    // ---- which key tiles this CTA visits -------------------------------------------------------------
    const int64_t first_qpos = q0 + m0, last_qpos = q0 + m0 + tok_in_tile - 1;
    const int64_t band_lo = (prm.window != 0 && first_qpos + 1 > (int64_t)prm.window) ? first_qpos + 1 - prm.window : 0;
    const int64_t last_lo = (prm.window != 0 && last_qpos + 1 > (int64_t)prm.window) ? last_qpos + 1 - prm.window : 0;
    int n_hist, n_tiles;
    int64_t hist_pos0 = 0, chunk_c0 = 0;
    if (TWO_SRC) {
        // history: positions [band_lo, q0) in the ring; chunk: positions [max(q0, band_lo), last_qpos]
        const int64_t h_lo = band_lo, h_hi = q0;  // half-open
        hist_pos0 = (h_lo / BLOCK_N) * BLOCK_N;
        n_hist = h_hi > h_lo ? (int)((h_hi - 1) / BLOCK_N - h_lo / BLOCK_N + 1) : 0;
        const int64_t c_lo = (band_lo > q0 ? band_lo - q0 : 0), c_hi = last_qpos - q0;  // inclusive chunk rows
        chunk_c0 = (c_lo / BLOCK_N) * BLOCK_N;
        n_tiles = n_hist + (int)(c_hi / BLOCK_N - c_lo / BLOCK_N + 1);
    } else {
        hist_pos0 = (band_lo / BLOCK_N) * BLOCK_N;
        n_hist = (int)(last_qpos / BLOCK_N - band_lo / BLOCK_N + 1);
        n_tiles = n_hist;
    }
    // gridDim.z pieces share a unit: piece z visits a contiguous run of its key tiles and leaves a partial
    // (unnormalised O, max, sum) that combine_pieces_kernel merges.  `it` below counts from the piece's
    // first tile, so barrier phases do not depend on the split.
    const int per_piece = (n_tiles + (int)gridDim.z - 1) / (int)gridDim.z;
    const int t_begin = min(n_tiles, (int)blockIdx.z * per_piece);
    n_tiles = min(n_tiles, t_begin + per_piece) - t_begin;
    auto tile_at = [&](int it) {
        Tile t;
        it += t_begin;
        if (it < n_hist) {
            t.src = 0;
            t.pos0 = hist_pos0 + (int64_t)it * BLOCK_N;
            t.row0 = (int)(TWO_SRC ? t.pos0 % prm.ring : t.pos0);
            t.lo = 0;
            t.hi = TWO_SRC ? q0 - 1 : INT64_MAX;
        } else {
            t.src = 1;
            const int64_t c = chunk_c0 + (int64_t)(it - n_hist) * BLOCK_N;
            t.pos0 = q0 + c;
            t.row0 = (int)c;
            t.lo = q0;
            t.hi = INT64_MAX;
        }
        return t;
    };

    // ---- set-up -----------------------------------------------------------------------------------------
    if (tid == 0) {
        for (int i = 0; i < KV_STAGES; i++) {
            mbar_init(&sm.full_k[i], 1);
            mbar_init(&sm.full_v[i], 1);
            mbar_init(&sm.s_ready[i], 1);
            mbar_init(&sm.p_ready[i], SOFTMAX_THREADS);
            mbar_init(&sm.pv_done[i], 1);
        }
        mbar_init(&sm.q_bar, 1);
        sm.abort = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(&sm.tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    bool failed = false;

    if (warp == LOAD_WARP) {
        // ======================= TMA loads =======================
        if ((tid & 31) == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k0);
            tma_prefetch_desc(&tm_v0);
            auto load_k = [&](int it) {
                const Tile t = tile_at(it);
                const int st = it % KV_STAGES;
                const CUtensorMap* mk = (TWO_SRC && t.src) ? &tm_k1 : &tm_k0;
                mbar_arrive_expect_tx(&sm.full_k[st], KV_TILE_BYTES);
                tma_load_3d(sm.k[st][0], mk, &sm.full_k[st], 0, kvh, t.row0);
                tma_load_3d(sm.k[st][1], mk, &sm.full_k[st], 64, kvh, t.row0);
            };
            auto load_v = [&](int it) {
                const Tile t = tile_at(it);
                const int st = it % KV_STAGES;
                const CUtensorMap* mv = (TWO_SRC && t.src) ? &tm_v1 : &tm_v0;
                mbar_arrive_expect_tx(&sm.full_v[st], KV_TILE_BYTES);
                tma_load_3d(sm.v[st][0], mv, &sm.full_v[st], 0, kvh, t.row0);
                tma_load_3d(sm.v[st][1], mv, &sm.full_v[st], 64, kvh, t.row0);
            };
            mbar_arrive_expect_tx(&sm.q_bar, Q_BYTES);
            tma_load_3d(sm.q[0], &tm_q, &sm.q_bar, 0, kvh * G, (int)m0);
            tma_load_3d(sm.q[1], &tm_q, &sm.q_bar, 64, kvh * G, (int)m0);
            if (n_tiles > 0) load_k(0);
            if (n_tiles > 1) load_k(1);
            if (n_tiles > 0) load_v(0);
            if (n_tiles > 1) load_v(1);
            for (int j = 0; j + 2 < n_tiles; ++j) {
                const int b = j % KV_STAGES;
                // K stage b is free once QK(j) has completed, V stage b once PV(j) has.
                mbar_wait(&sm.s_ready[b], (j / 2) & 1, prm.status, 411, failed, 100);
                if (failed) break;  // never write into a stage that may still be read
                load_k(j + 2);
                mbar_wait(&sm.pv_done[b], (j / 2) & 1, prm.status, 412, failed, 100);
                if (failed) break;
                load_v(j + 2);
            }
        }
    } else if (warp == MMA_WARP) {
        // ======================= MMA issue =======================
        if ((tid & 31) == 0) {
            constexpr uint32_t IDESC_QK = umma_idesc_f16(BLOCK_M, BLOCK_N, 0, 0);
            constexpr uint32_t IDESC_PV = umma_idesc_f16(BLOCK_M, HD, 0, 1);
            // Operand descriptors are built once; a step of 32 bytes along K (or of 16 keys of V) is an add to the
            // descriptor's address field (bytes >> 4).  Building them per instruction costs the issuing thread more
            // cycles than the tensor pipe needs for the instruction.
            const uint64_t dq[2] = {umma_desc_sw128(smem_u32(sm.q[0]), 16, 1024), umma_desc_sw128(smem_u32(sm.q[1]), 16, 1024)};
            const uint64_t dk[2][2] = {{umma_desc_sw128(smem_u32(sm.k[0][0]), 16, 1024), umma_desc_sw128(smem_u32(sm.k[0][1]), 16, 1024)},
                                       {umma_desc_sw128(smem_u32(sm.k[1][0]), 16, 1024), umma_desc_sw128(smem_u32(sm.k[1][1]), 16, 1024)}};
            const uint64_t dv[2] = {umma_desc_sw128(smem_u32(sm.v[0][0]), HALF_TILE, 1024), umma_desc_sw128(smem_u32(sm.v[1][0]), HALF_TILE, 1024)};
            // S[j % 2] = Q K(j)^T: 8 MMAs of K = 16, once K(j) has landed.
            auto issue_qk = [&](int j) {
                const int b = j % KV_STAGES;
                mbar_wait(&sm.full_k[b], (j / KV_STAGES) & 1, prm.status, 402, failed);
                if (failed) return;
                tc_fence_after_sync();
                const uint64_t k0 = b ? dk[1][0] : dk[0][0], k1 = b ? dk[1][1] : dk[0][1];
                const uint32_t d = tmem + TMEM_S + b * BLOCK_N;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(d, dq[0] + 2 * kk, k0 + 2 * kk, IDESC_QK, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(d, dq[1] + 2 * kk, k1 + 2 * kk, IDESC_QK, 1u);
                umma_commit(&sm.s_ready[b]);
            };
            mbar_wait(&sm.q_bar, 0, prm.status, 401, failed);
            if (n_tiles > 0) issue_qk(0);
            if (n_tiles > 1) issue_qk(1);
            for (int j = 0; j < n_tiles; ++j) {
                const int b = j % KV_STAGES;
                mbar_wait(&sm.p_ready[b], (j / 2) & 1, prm.status, 403, failed);
                mbar_wait(&sm.full_v[b], (j / KV_STAGES) & 1, prm.status, 405, failed);
                if (failed) break;
                tc_fence_after_sync();
                {
                    // P(j) lives in the first 32 columns of S[b] (packed f16 pairs), written by the softmax warps
                    const uint64_t v0 = b ? dv[1] : dv[0];
                    const uint32_t pa = tmem + TMEM_S + b * BLOCK_N;
                    umma_f16_ts(tmem + TMEM_O, pa, v0, IDESC_PV, j ? 1u : 0u);
#pragma unroll
                    for (int kk = 1; kk < 4; kk++) umma_f16_ts(tmem + TMEM_O, pa + kk * 8, v0 + 128 * kk, IDESC_PV, 1u);
                }
                umma_commit(&sm.pv_done[b]);
                if (j + 2 < n_tiles) {
                    // S[b] may be overwritten: the softmax warps read it before they produced P(j), waited for above
                    issue_qk(j + 2);
                }
            }
        }
    } else {
        // ======================= softmax: row r of the tile <-> TMEM lane r <-> thread r =======================
        // token m0 + r/2, query head kvh*2 + r%2
        const int r = tid;
        const uint32_t tok = m0 + (uint32_t)(r >> 1);
        const int64_t qpos = q0 + tok;
        const int64_t row_lo = (prm.window != 0 && qpos + 1 > (int64_t)prm.window) ? qpos + 1 - prm.window : 0;
        const float scale2 = prm.scale * 1.4426950408889634f;  // > 0 (checked on the host)
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        float m_run = NEG_SENTINEL, l_run = 0.0f;

        for (int it = 0; it < n_tiles; ++it) {
            const int b = it % 2;
            const Tile t = tile_at(it);
            mbar_wait(&sm.s_ready[b], (it / 2) & 1, prm.status, 404, failed);
            tc_fence_after_sync();
            float v[64];
            {
                uint32_t a0[32], a1[32];
                tmem_ld_32x32b_x32(lane_addr + TMEM_S + b * BLOCK_N, a0);
                tmem_ld_32x32b_x32(lane_addr + TMEM_S + b * BLOCK_N + 32, a1);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    v[j] = __uint_as_float(a0[j]);
                    v[32 + j] = __uint_as_float(a1[j]);
                }
            }

            // A tile needs per-element masks only where it crosses a band edge or a source boundary.
            const bool tile_masked = t.pos0 + BLOCK_N - 1 > first_qpos || t.pos0 < last_lo || t.pos0 < t.lo || t.pos0 + BLOCK_N - 1 > t.hi;
            if (tile_masked) {
                const int64_t hi = min(qpos, t.hi), lo = max(row_lo, t.lo);
#pragma unroll
                for (int j = 0; j < 64; j++) {
                    const int64_t pos = t.pos0 + j;
                    if (pos < lo || pos > hi) v[j] = -INFINITY;
                }
            }
            // row max of the raw scores on four independent chains of three-input max; scale2 > 0
            // commutes with max
            float mx4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
            for (int j = 4; j < 64; j += 2) mx4[(j >> 1) & 3] = max3(mx4[(j >> 1) & 3], v[j], v[j + 1]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale2;
            const bool grow = mx > m_run + RESCALE_T;
            float corr = 1.0f;
            if (grow) {
                corr = ex2(m_run - mx);
                m_run = mx;
                l_run *= corr;
            }
            // p = 2^(s * scale2 - m) with the multiply-add and the running sums on packed f32x2 pipes
            const float2 sc2 = make_float2(scale2, scale2), neg_m = make_float2(-m_run, -m_run);
            uint32_t pk[32];
            float2 ls4[4] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float2 x = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), sc2, neg_m);
                const float2 pp = make_float2(ex2(x.x), ex2(x.y));
                ls4[j & 3] = __fadd2_rn(ls4[j & 3], pp);  // l in f32 from the unrounded p (attn_prefill_global_flash_sp.wgsl:147-156)
                pk[j] = pack_half2(pp.x, pp.y);
            }
            l_run += ((ls4[0].x + ls4[0].y) + (ls4[1].x + ls4[1].y)) + ((ls4[2].x + ls4[2].y) + (ls4[3].x + ls4[3].y));

            // O is rescaled where a row's max moved (rare after the first tiles), and only once P V of the
            // previous tile has completed.  P(it) itself needs no such wait: it goes into S[b], which the
            // tensor pipe next touches with P V(it).  (Most tiles skip this wait; its parity stays
            // unambiguous because pv_done[b ^ 1] is next committed by P V(it + 1), which needs this
            // thread's P(it + 1).)
            if (it > 0 && __any_sync(0xffffffffu, grow)) {
                mbar_wait(&sm.pv_done[b ^ 1], ((it - 1) / 2) & 1, prm.status, 407, failed);
                tc_fence_after_sync();
                {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint32_t o[32];
                        tmem_ld_32x32b_x32(lane_addr + TMEM_O + 32 * c, o);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
                        tmem_st_32x32b_x32(lane_addr + TMEM_O + 32 * c, o);
                    }
                    tc_wait_st();
                }
            }
            // Rows of the V tile that hold no key of this problem (past the last query's position, or past the end
            // of the history source) are zeroed before P V reads them: their P is 0, but 0 times a stale Inf or NaN
            // in a caller's over-allocated buffer would not be.  Only the last tile of a source can have such rows.
            {
                const int64_t hi_valid = min(t.hi, q0 + (int64_t)prm.m_tokens - 1);
                if (t.pos0 + BLOCK_N - 1 > hi_valid) {  // uniform over the CTA
                    mbar_wait(&sm.full_v[b], (it / KV_STAGES) & 1, prm.status, 409, failed);
                    if (r < BLOCK_N && t.pos0 + r > hi_valid) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            uint4* row = reinterpret_cast<uint4*>(sm.v[b][h] + r * 128);
#pragma unroll
                            for (int i = 0; i < 8; i++) row[i] = make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                    fence_proxy_async_smem();  // generic-proxy writes, read next by the tensor pipe
                }
            }
            // P row r goes back into tensor memory over the first half of S[b] (this thread has S in
            // registers; Q K^T of tile it + 2 overwrites the buffer only after P V of this tile, because the
            // tensor pipe runs in order).
            tmem_st_32x32b_x32(lane_addr + TMEM_S + b * BLOCK_N, pk);
            tc_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_ready[b]);
        }
        // the tensor pipe completes in order: the last P V done means all of them are
        if (n_tiles > 0) mbar_wait(&sm.pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) / 2) & 1, prm.status, 408, failed);
        tc_fence_after_sync();

        // ---- epilogue: out = O / l, or this piece's partial.  The TMEM loads are warp-wide, so every thread
        // takes part and only the stores are predicated (rows past the end of the chunk are not written). ----
        const bool live = (uint32_t)(r >> 1) < tok_in_tile;
        const size_t row = (size_t)(live ? tok : m0) * (prm.n_kv * G) + kvh * G + (r & 1);
        const bool whole = gridDim.z == 1;
        const float mul = whole ? 1.0f / l_run : 1.0f;
        float* orow = whole ? prm.out + row * HD : prm.part_acc + (row * gridDim.z + blockIdx.z) * HD;
        if (!whole && live) *reinterpret_cast<float2*>(prm.part_ml + (row * gridDim.z + blockIdx.z) * 2) = make_float2(m_run, l_run);
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t o[32];
            if (n_tiles > 0) {  // uniform over the CTA
                tmem_ld_32x32b_x32(lane_addr + TMEM_O + 32 * c, o);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) o[j] = 0u;  // an empty piece: m = sentinel, l = 0, O = 0
            }
            if (live) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<float4*>(orow + 32 * c + 4 * j) =
                        make_float4(__uint_as_float(o[4 * j]) * mul, __uint_as_float(o[4 * j + 1]) * mul,
                                    __uint_as_float(o[4 * j + 2]) * mul, __uint_as_float(o[4 * j + 3]) * mul);
            }
        }
    }
    // A wait that ran out leaves copies and MMAs of this CTA in flight that nobody will wait for: give them
    // a bounded time to land before the shared and tensor memory they target is handed to the next CTA.
    if (failed) sm.abort = 1;
    tc_fence_before_sync();
    __syncthreads();
    if (*(volatile uint32_t*)&sm.abort != 0u) {
        for (int i = 0; i < 50; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// Merge the pieces of every row: out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p, pieces in index
// order (fixed order => bit-identical reruns).  One warp per row, lane = 4 dims.
constexpr int MAX_PIECES = 16;
__global__ void __launch_bounds__(256) combine_pieces_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                             float* __restrict__ out, uint32_t rows, uint32_t pieces)
{
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float m[MAX_PIECES], l[MAX_PIECES];
    float big = NEG_SENTINEL;
#pragma unroll
    for (int p = 0; p < MAX_PIECES; p++) {
        if (p < (int)pieces) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)row * pieces + p) * 2);
            m[p] = ml.x;
            l[p] = ml.y;
            big = fmaxf(big, ml.x);
        }
    }
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float den = 0.0f;
#pragma unroll
    for (int p = 0; p < MAX_PIECES; p++) {
        if (p < (int)pieces) {
            const float w = l[p] > 0.0f ? ex2(m[p] - big) : 0.0f;
            const float4 a = *reinterpret_cast<const float4*>(part_acc + ((size_t)row * pieces + p) * HD + lane * 4);
            acc.x = fmaf(w, a.x, acc.x);
            acc.y = fmaf(w, a.y, acc.y);
            acc.z = fmaf(w, a.z, acc.z);
            acc.w = fmaf(w, a.w, acc.w);
            den = fmaf(w, l[p], den);
        }
    }
    const float inv = 1.0f / den;
    *reinterpret_cast<float4*>(out + (size_t)row * HD + lane * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// Scratch for the pieces: one growing allocation per (device, stream), made outside stream capture only.
// Launches on one stream are ordered, so they can share a block; launches on different streams may overlap
// and get a block each.  Blocks are never freed before the process ends: work in flight, or a recorded
// graph, may still point at them.
struct PieceScratch {
    float* ptr = nullptr;
    size_t bytes = 0;
};
std::mutex g_piece_mutex;
std::map<std::pair<int, cudaStream_t>, PieceScratch> g_piece_scratch;

// How many pieces to cut every unit's key range into.  The host does not know kv_len (it lives in the
// step buffer), so the choice rests on the grid alone: with `units` equal CTAs on `slots` resident
// places the last wave is ceil(w) - w empty; more pieces make the waves finer.  The K buffer's row
// count bounds kv_len from above and keeps tiny problems whole.
int choose_pieces(size_t units, int slots, size_t kv_rows_bound)
{
    if (const char* e = getenv("SGB_FLASH_PIECES")) {
        const int v = atoi(e);
        if (v >= 1 && v <= MAX_PIECES) return v;
    }
    const size_t max_by_len = kv_rows_bound / 2048;  // at least 2048 keys per piece
    int best = 1;
    double best_eff = 0.0;
    for (int p = 1; p <= MAX_PIECES && (p == 1 || (size_t)p <= max_by_len); p++) {
        const double w = (double)units * p / slots;
        const double eff = w / ceil(w) - 0.004 * (p - 1);  // each extra piece costs a partial write + read
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = p;
        }
    }
    return best;
}

struct PushScaleWindow {
    float scale;
    uint32_t window;
};
struct PushScalePage {
    float scale;
    uint32_t page;
};

int encode_qkv_map(const LaunchArgs& a, CUtensorMap* tm, const BufView& buf, uint64_t heads, uint32_t box_heads,
                   uint32_t box_rows, const char* what)
{
    const uint64_t rows = buf.bytes / (heads * HD * 2);
    if (rows == 0) return fail_validation(a, std::string(what) + ": buffer holds no complete row");
    if (reinterpret_cast<uintptr_t>(buf.ptr) & 15) return fail_validation(a, std::string(what) + ": buffer must be 16-byte aligned");
    const uint64_t dims[3] = {HD, heads, rows};
    const uint64_t strides[2] = {HD * 2, heads * HD * 2};
    const uint32_t box[3] = {64, box_heads, box_rows};
    return encode_tensor_map(a, tm, 1, 3, buf.ptr, dims, strides, box, 3);
}

template <bool TWO_SRC>
int run_flash(const LaunchArgs& a, const BufView& q, const BufView& k0, const BufView& v0, const BufView* k1, const BufView* v1,
              const BufView& out, const BufView& step, uint32_t n_kv, uint32_t m_tokens, float scale, uint32_t window,
              uint32_t ring)
{
    if (n_kv == 0 || m_tokens == 0) return fail_validation(a, "flash prefill: groups must be [kv heads, query tokens]");
    if (!(scale > 0.0f)) return fail_validation(a, "flash prefill: the softmax scale must be positive");
    const size_t n_q = (size_t)n_kv * G;
    if (q.bytes < (size_t)m_tokens * n_q * HD * 2) return fail_validation(a, "flash prefill: q buffer too small");
    if (out.bytes < (size_t)m_tokens * n_q * HD * 4) return fail_validation(a, "flash prefill: out buffer too small");
    if (step.bytes < 16) return fail_validation(a, "flash prefill: the step buffer holds 4 x u32");
    if (reinterpret_cast<uintptr_t>(out.ptr) & 15) return fail_validation(a, "flash prefill: out must be 16-byte aligned");
    CUtensorMap tq, tk0, tv0, tk1, tv1;
    if (int r = encode_qkv_map(a, &tq, BufView{q.ptr, (size_t)m_tokens * n_q * HD * 2}, n_q, G, BLOCK_TOK, "q")) return r;
    if (int r = encode_qkv_map(a, &tk0, k0, n_kv, 1, BLOCK_N, "k")) return r;
    if (int r = encode_qkv_map(a, &tv0, v0, n_kv, 1, BLOCK_N, "v")) return r;
    if (TWO_SRC) {
        if (k0.bytes < (size_t)ring * n_kv * HD * 2 || v0.bytes < (size_t)ring * n_kv * HD * 2)
            return fail_validation(a, "flash prefill: ring buffers smaller than the ring");
        if (k1->bytes < (size_t)m_tokens * n_kv * HD * 2 || v1->bytes < (size_t)m_tokens * n_kv * HD * 2)
            return fail_validation(a, "flash prefill: chunk K/V hold fewer than M rows");
        if (int r = encode_qkv_map(a, &tk1, *k1, n_kv, 1, BLOCK_N, "k_chunk")) return r;
        if (int r = encode_qkv_map(a, &tv1, *v1, n_kv, 1, BLOCK_N, "v_chunk")) return r;
    } else {
        tk1 = tk0;
        tv1 = tv0;
    }
    const size_t smem = sizeof(FlashSmem);
    {
        static std::mutex attr_mutex;
        static bool attr_set[2][64] = {};
        std::lock_guard<std::mutex> lock(attr_mutex);
        if (a.device < 64 && !attr_set[TWO_SRC][a.device]) {
            if (int r = check_cuda(a, cudaFuncSetAttribute(flash_prefill_kernel<TWO_SRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                   "cudaFuncSetAttribute(flash_prefill)"))
                return r;
            attr_set[TWO_SRC][a.device] = true;
        }
    }
    const size_t k_rows = k0.bytes / ((size_t)n_kv * HD * 2);
    const uint32_t q_tiles = (m_tokens + BLOCK_TOK - 1) / BLOCK_TOK;
    const size_t rows = (size_t)m_tokens * n_q;
    int pieces = TWO_SRC ? 1 : choose_pieces((size_t)q_tiles * n_kv, 2 * a.sm_count, k_rows);
    float* part_acc = nullptr;
    float* part_ml = nullptr;
    if (pieces > 1) {
        const size_t need = rows * pieces * (HD + 2) * sizeof(float);
        std::lock_guard<std::mutex> lock(g_piece_mutex);
        PieceScratch& sc = g_piece_scratch[std::make_pair(a.device, a.stream)];
        if (sc.bytes < need) {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(a.stream, &cap);
            if (cap != cudaStreamCaptureStatusNone) {
                pieces = 1;  // no allocation while a graph is being recorded: run whole units
            } else {
                // A block that no longer suffices is kept, not freed: a recorded graph may still point at it.
                const size_t want = need > 2 * sc.bytes ? need : 2 * sc.bytes;  // geometric growth bounds what is left behind
                sc = PieceScratch{};
                if (cudaMalloc(&sc.ptr, want) == cudaSuccess) {
                    sc.bytes = want;
                } else {
                    (void)cudaGetLastError();
                    sc = PieceScratch{};
                    pieces = 1;  // not enough memory for partials: run whole units
                }
            }
        }
        if (pieces > 1) {
            part_acc = sc.ptr;
            part_ml = sc.ptr + rows * pieces * HD;
        }
    }
    // Heads per group: as many as keep the group's f16 K and V (an upper bound: the K buffer's rows) within about three
    // quarters of the 126 MB L2, a divisor of the head count.  Measured: all 16 heads of an 8192-token problem (67 MB)
    // as one group 1056 TFLOP/s against 981 head by head; a 131072-token cache (67 MB per head) head by head 1094
    // against 1040 with all heads in one group.
    uint32_t head_group = 1;
    {
        const size_t per_head = k_rows * HD * 2 * 2;
        for (uint32_t g = 1; g <= n_kv; g++)
            if (n_kv % g == 0 && g * per_head <= (size_t)96 << 20) head_group = g;
        if (const char* e = getenv("SGB_FLASH_HEAD_GROUP")) {  // tuning and test aid; the results do not depend on it
            const int v = atoi(e);
            if (v >= 1 && (uint32_t)v <= n_kv && n_kv % (uint32_t)v == 0) head_group = (uint32_t)v;
        }
    }
    FlashParams prm{(const uint32_t*)step.ptr, (float*)out.ptr, part_acc, part_ml, a.status, m_tokens, n_kv, window, ring, scale, head_group};
    const dim3 grid(q_tiles * n_kv, 1, pieces);
    flash_prefill_kernel<TWO_SRC><<<grid, FLASH_THREADS, smem, a.stream>>>(tq, tk0, tv0, tk1, tv1, prm);
    ++*a.launches;
    if (int r = check_cuda(a, cudaGetLastError(), "attn_prefill_flash")) return r;
    if (pieces > 1) {
        combine_pieces_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, a.stream>>>(part_acc, part_ml, (float*)out.ptr, (uint32_t)rows,
                                                                              (uint32_t)pieces);
        ++*a.launches;
        return check_cuda(a, cudaGetLastError(), "attn_prefill_flash combine");
    }
    return 0;
}

}  // namespace

// attn_prefill_flash_f16_d128: q, k, v, out f32, step.  push {scale, window}.  grid [KV, M].
int launch_prefill_flash_f16_d128(const LaunchArgs& a)
{
    const PushScaleWindow p = *(const PushScaleWindow*)a.push;
    return run_flash<false>(a, a.b[0], a.b[1], a.b[2], nullptr, nullptr, a.b[3], a.b[4], a.groups[0], a.groups[1], p.scale,
                            p.window, 0);
}

// attn_prefill_sliding_ring_flash_d128: q, k_ring, v_ring, k_chunk, v_chunk, out f32, step.  push {scale}.
int launch_prefill_sliding_ring_flash_d128(const LaunchArgs& a)
{
    const float scale = *(const float*)a.push;
    return run_flash<true>(a, a.b[0], a.b[1], a.b[2], &a.b[3], &a.b[4], a.b[5], a.b[6], a.groups[0], a.groups[1], scale, 1024,
                           1024);
}

// attn_prefill_paged_q8kv_flash_d128: q, k_quants, k_scales, v_quants, v_scales, page_table,
// k_lin, v_lin (f16 scratch, rows x KV x 128), out f32, step.  push {scale, page}.  grid [KV, M].
int launch_prefill_paged_q8kv_flash_d128(const LaunchArgs& a)
{
    const PushScalePage p = *(const PushScalePage*)a.push;
    const uint32_t n_kv = a.groups[0];
    if (n_kv == 0 || p.page == 0) return fail_validation(a, "paged flash prefill: kv heads and page must be > 0");
    const uint32_t row_len = n_kv * HD;
    if (int r = run_kv_dequant_paged(a, a.b[2], a.b[1], a.b[5], a.b[6], a.b[9], row_len, p.page)) return r;
    if (int r = run_kv_dequant_paged(a, a.b[4], a.b[3], a.b[5], a.b[7], a.b[9], row_len, p.page)) return r;
    return run_flash<false>(a, a.b[0], a.b[6], a.b[7], nullptr, nullptr, a.b[8], a.b[9], n_kv, a.groups[1], p.scale, 0, 0);
}

}  // namespace sgb
