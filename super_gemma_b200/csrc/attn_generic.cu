// Scalar (CUDA-core) attention kernels: every reference-shaped registry name, and the d128 cases
// that are too small for a tensor-core tile (sliding decode, 4-token verify over the ring, the
// 512-token sliding prefill).  They follow the reference's streaming-softmax statement per key
// (attn_decode_sliding.wgsl:84-107 and its siblings) with f32 math, one warp per key and the four
// warps of a block merged in a fixed order, so reruns are bit-identical.
#include "attn_merge.cuh"
#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int GEN_THREADS = 128;
constexpr int GEN_WARPS = GEN_THREADS / 32;

// FMT_Q8: value = f32(scale) * f32(q), unrounded (attn_decode_global_q8k.wgsl:82, and the exact product the
// int8 path of attn_prefill_global_flash_sp_iq.wgsl forms).  FMT_Q8_F16: the same product rounded to f16,
// the value attn_prefill_global_flash_sp_q8.wgsl:104 stages in shared memory (= kv_dequant_q8).
enum : int { FMT_F16 = 0, FMT_Q8 = 1, FMT_Q8_F16 = 2 };

struct KvOperand {
    const void* data;           // f16 rows, or int8 quants
    const __half* scales;       // Q8_0 scales (FMT_Q8 only)
    const uint32_t* page_table; // nullptr = linear
    uint32_t table_len;
    uint32_t page;
    size_t rows;                // rows the buffer holds (bounds checks)
};

template <int DPL>
__device__ __forceinline__ void load_f16(const __half* p, float (&out)[DPL])
{
    if constexpr (DPL % 8 == 0) {
#pragma unroll
        for (int i = 0; i < DPL / 8; i++) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + i);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                out[i * 8 + 2 * j] = f.x;
                out[i * 8 + 2 * j + 1] = f.y;
            }
        }
    } else {
        static_assert(DPL % 4 == 0, "lanes own 4 or more dims");
#pragma unroll
        for (int i = 0; i < DPL / 4; i++) {
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(p) + i);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const float2 f = __half22float2(h[j]);
                out[i * 4 + 2 * j] = f.x;
                out[i * 4 + 2 * j + 1] = f.y;
            }
        }
    }
}

// kk = f32(scale) * f32(q), not re-rounded (attn_decode_global_q8k.wgsl:82).  A lane's DPL dims
// (DPL <= 32, d0 a multiple of DPL) lie inside one 32-value block.
template <int DPL>
__device__ __forceinline__ void load_q8(const int8_t* q, const __half* scales, int d0, float (&out)[DPL])
{
    const float s = __half2float(__ldg(scales + d0 / 32));
#pragma unroll
    for (int i = 0; i < DPL / 4; i++) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(q) + i);
        out[4 * i] = __fmul_rn(s, (float)(int8_t)(w & 0xFF));
        out[4 * i + 1] = __fmul_rn(s, (float)(int8_t)((w >> 8) & 0xFF));
        out[4 * i + 2] = __fmul_rn(s, (float)(int8_t)((w >> 16) & 0xFF));
        out[4 * i + 3] = __fmul_rn(s, (float)(int8_t)(w >> 24));
    }
}

// One K or V row slice for this lane.  `row` is already physical.
template <int HD, int FMT, int DPL>
__device__ __forceinline__ void load_row(const KvOperand& op, size_t row, int kvh, int n_kv, int d0, float (&out)[DPL])
{
    const size_t base = (row * n_kv + kvh) * HD;
    if constexpr (FMT == FMT_F16) {
        load_f16<DPL>(reinterpret_cast<const __half*>(op.data) + base + d0, out);
    } else {
        load_q8<DPL>(reinterpret_cast<const int8_t*>(op.data) + base + d0, op.scales + (row * n_kv + kvh) * (HD / 32), d0,
                     out);
        if constexpr (FMT == FMT_Q8_F16) {
#pragma unroll
            for (int d = 0; d < DPL; d++) out[d] = __half2float(__float2half_rn(out[d]));
        }
    }
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int G, int DPL>
struct Stream {
    float m[G], l[G], acc[G][DPL];
    __device__ __forceinline__ void init()
    {
#pragma unroll
        for (int g = 0; g < G; g++) {
            m[g] = NEG_SENTINEL;
            l[g] = 0.0f;
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[g][d] = 0.0f;
        }
    }
    // attn_decode_sliding.wgsl:92-106 for head g
    __device__ __forceinline__ void step(int g, const float (&qr)[DPL], const float (&kk)[DPL], const float (&vv)[DPL],
                                         float scale)
    {
        float dot = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; d++) dot = fmaf(qr[d], kk[d], dot);
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m[g], s);
        const float corr = __expf(m[g] - m_new);
        const float w = __expf(s - m_new);
        l[g] = l[g] * corr + w;
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[g][d] = acc[g][d] * corr + w * vv[d];
        m[g] = m_new;
    }
};

// Merge the four warps' streaming states in warp order 0,1,2,3 through shared memory, leaving the
// result in warp 0's registers.  sm_acc holds G*HD floats, sm_ml holds 2*G floats.
template <int HD, int G, int DPL>
__device__ __forceinline__ void merge_warps(Stream<G, DPL>& st, float* sm_acc, float* sm_ml, int warp, int lane, int d0)
{
    for (int w = 1; w < GEN_WARPS; w++) {
        __syncthreads();
        if (warp == w) {
#pragma unroll
            for (int g = 0; g < G; g++) {
#pragma unroll
                for (int d = 0; d < DPL; d++) sm_acc[g * HD + d0 + d] = st.acc[g][d];
                if (lane == 0) {
                    sm_ml[2 * g] = st.m[g];
                    sm_ml[2 * g + 1] = st.l[g];
                }
            }
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float ms = sm_ml[2 * g], ls = sm_ml[2 * g + 1];
                const float m_new = fmaxf(st.m[g], ms);
                const float ca = __expf(st.m[g] - m_new), cb = __expf(ms - m_new);
#pragma unroll
                for (int d = 0; d < DPL; d++) st.acc[g][d] = st.acc[g][d] * ca + sm_acc[g * HD + d0 + d] * cb;
                st.l[g] = st.l[g] * ca + ls * cb;
                st.m[g] = m_new;
            }
        }
    }
}

__device__ __forceinline__ bool resolve_row(const KvOperand& op, size_t t, size_t& row, uint32_t* status, uint32_t site)
{
    row = t;
    if (op.page_table != nullptr) {
        const size_t p = t / op.page;
        if (p >= op.table_len) {
            report_error(status, DEV_ERR_BOUNDS, site, (uint32_t)p, op.table_len);
            return false;
        }
        row = (size_t)op.page_table[p] * op.page + t % op.page;
    }
    if (row >= op.rows) {
        report_error(status, DEV_ERR_BOUNDS, site + 1, (uint32_t)row, (uint32_t)op.rows);
        return false;
    }
    return true;
}

// Split-K decode partials.  Grid (kv head, split, query token); the reference's grid is the first
// two (attn_decode_sliding.wgsl:53-62).  part row = i * H + qh.
template <int HD, int G, int KFMT, int VFMT>
__global__ void __launch_bounds__(GEN_THREADS) decode_generic_kernel(const __half* __restrict__ q, KvOperand kop, KvOperand vop,
                                                                     float* __restrict__ part,
                                                                     const uint32_t* __restrict__ step, int step_slot,
                                                                     uint32_t n_splits, float scale, uint32_t* status)
{
    constexpr int DPL = HD / 32;
    __shared__ float sm_acc[G * HD];
    __shared__ float sm_ml[2 * G];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = blockIdx.x, n_kv = gridDim.x, split = blockIdx.y;
    const uint32_t i = blockIdx.z, m_q = gridDim.z;
    const int n_q = n_kv * G;
    const int d0 = lane * DPL;

    const uint32_t kv_len = step[step_slot];
    const uint32_t chunk = (kv_len + n_splits - 1) / n_splits;
    const uint32_t t_begin = min((uint32_t)split * chunk, kv_len);
    uint32_t t_end = min(t_begin + chunk, kv_len);
    // query i of m_q sees keys t <= kv_len - m_q + i  (m_q = 1: every key)
    const uint32_t vis_end = kv_len + i >= m_q ? kv_len + i - m_q + 1 : 0;
    t_end = min(t_end, vis_end);

    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++) load_f16<DPL>(q + ((size_t)i * n_q + kvh * G + g) * HD + d0, qr[g]);

    Stream<G, DPL> st;
    st.init();
    for (uint32_t t = t_begin + warp; t < t_end; t += GEN_WARPS) {
        size_t krow, vrow;
        if (!resolve_row(kop, t, krow, status, 201) || !resolve_row(vop, t, vrow, status, 203)) break;
        float kk[DPL], vv[DPL];
        load_row<HD, KFMT, DPL>(kop, krow, kvh, n_kv, d0, kk);
        load_row<HD, VFMT, DPL>(vop, vrow, kvh, n_kv, d0, vv);
#pragma unroll
        for (int g = 0; g < G; g++) st.step(g, qr[g], kk, vv, scale);
    }
    merge_warps<HD, G, DPL>(st, sm_acc, sm_ml, warp, lane, d0);
    if (warp == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float* row = part + (((size_t)i * n_q + kvh * G + g) * n_splits + split) * (HD + 2);
#pragma unroll
            for (int d = 0; d < DPL; d++) row[d0 + d] = st.acc[g][d];
            if (lane == 0) {
                row[HD] = st.m[g];
                row[HD + 1] = st.l[g];
            }
        }
    }
}

// Split-K combine (attn_reduce.wgsl:29-56): the splits of a row in ascending order with a running
// maximum, the reference's own op order (merge_splits_running).  Grid = rows, HD / 2 threads, two dims each.
// OUT_MODE 0: f16(acc/l) (the reference), 1: f32 acc/l, 2: merged (acc, m, l) as f32[HD+2].
// split_major = 0: part[(row*n + s)*(HD+2)]; 1: part[(s*rows + row)*(HD+2)] (per-rank blocks).
constexpr int REDUCE_MAX_SPLITS = 1024;

template <int HD, int OUT_MODE>
__global__ void __launch_bounds__(HD / 2) reduce_kernel(const float* __restrict__ part, void* __restrict__ out, uint32_t n_splits,
                                                       int split_major)
{
    const size_t row = blockIdx.x, rows = gridDim.x;
    const int d0 = 2 * threadIdx.x;
    pdl_wait();  // the partials come from the kernel before this one
    pdl_launch_dependents();
    const size_t s_stride = split_major ? rows * (HD + 2) : (size_t)(HD + 2);
    const float* base = part + (split_major ? row : row * n_splits) * (HD + 2);
    float acc[2];
    const MergeState st = merge_splits_running<HD, 2, 3>(base, s_stride, n_splits, d0, acc);  // up to 96 splits in one latency
    if constexpr (OUT_MODE == 2) {
        float* o = reinterpret_cast<float*>(out) + row * (HD + 2);
        *reinterpret_cast<float2*>(o + d0) = make_float2(acc[0], acc[1]);
        if (threadIdx.x == 0) *reinterpret_cast<float2*>(o + HD) = make_float2(st.m, st.l);
    } else if constexpr (OUT_MODE == 0) {
        reinterpret_cast<__half2*>(out)[(row * HD + d0) / 2] = __floats2half2_rn(acc[0] / st.l, acc[1] / st.l);
    } else {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + row * HD + d0) = make_float2(acc[0] / st.l, acc[1] / st.l);
    }
}

// Streaming prefill.  Grid (kv head, query token).  TWO_RANGE: history [t_begin, min(q0, qpos+1))
// from `hist` at row t % ring, then chunk rows [max(q0, t_begin) - q0, i] from `chunk`
// (attn_prefill_sliding_ring.wgsl:88-140); otherwise one linear range [t_begin, qpos] from `hist`
// (attn_prefill_sliding.wgsl:53-57,78 / attn_prefill_global.wgsl:53,74).  window 0 = none.
// QFMT = FMT_Q8: q holds int8 quants [M x H x HD] with f16 scales q_scales [M x H x HD/32]
// (attn_prefill_global_flash_sp_iq.wgsl:24-25).
template <int HD, int G, int KFMT, int VFMT, int TWO_RANGE, int OUT_F32, int QFMT = FMT_F16>
__global__ void __launch_bounds__(GEN_THREADS) prefill_generic_kernel(const void* __restrict__ q, const __half* __restrict__ q_scales,
                                                                      KvOperand k_hist, KvOperand v_hist, KvOperand k_chunk,
                                                                      KvOperand v_chunk, void* __restrict__ out,
                                                                      const uint32_t* __restrict__ step, uint32_t window,
                                                                      uint32_t ring, float scale, uint32_t* status)
{
    constexpr int DPL = HD / 32;
    __shared__ float sm_acc[G * HD];
    __shared__ float sm_ml[2 * G];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = blockIdx.x, n_kv = gridDim.x;
    const uint32_t i = blockIdx.y;
    const int n_q = n_kv * G;
    const int d0 = lane * DPL;
    const uint32_t q0 = step[STEP_Q0];
    const uint32_t qpos = q0 + i;
    const uint32_t t_begin = (window != 0 && qpos + 1 > window) ? qpos + 1 - window : 0;

    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const size_t qrow = (size_t)i * n_q + kvh * G + g;
        if constexpr (QFMT == FMT_F16)
            load_f16<DPL>(reinterpret_cast<const __half*>(q) + qrow * HD + d0, qr[g]);
        else
            load_q8<DPL>(reinterpret_cast<const int8_t*>(q) + qrow * HD + d0, q_scales + qrow * (HD / 32), d0, qr[g]);
    }

    Stream<G, DPL> st;
    st.init();
    const uint32_t hist_end = TWO_RANGE ? min(q0, qpos + 1) : qpos + 1;
    for (uint32_t t = t_begin + warp; t < hist_end; t += GEN_WARPS) {
        const size_t lt = ring ? t % ring : t;
        size_t krow, vrow;
        if (!resolve_row(k_hist, lt, krow, status, 211) || !resolve_row(v_hist, lt, vrow, status, 213)) break;
        float kk[DPL], vv[DPL];
        load_row<HD, KFMT, DPL>(k_hist, krow, kvh, n_kv, d0, kk);
        load_row<HD, VFMT, DPL>(v_hist, vrow, kvh, n_kv, d0, vv);
#pragma unroll
        for (int g = 0; g < G; g++) st.step(g, qr[g], kk, vv, scale);
    }
    if (TWO_RANGE) {
        const uint32_t c_begin = t_begin > q0 ? t_begin - q0 : 0;
        for (uint32_t c = c_begin + warp; c <= i; c += GEN_WARPS) {
            size_t krow, vrow;
            if (!resolve_row(k_chunk, c, krow, status, 215) || !resolve_row(v_chunk, c, vrow, status, 217)) break;
            float kk[DPL], vv[DPL];
            load_row<HD, FMT_F16, DPL>(k_chunk, krow, kvh, n_kv, d0, kk);
            load_row<HD, FMT_F16, DPL>(v_chunk, vrow, kvh, n_kv, d0, vv);
#pragma unroll
            for (int g = 0; g < G; g++) st.step(g, qr[g], kk, vv, scale);
        }
    }
    merge_warps<HD, G, DPL>(st, sm_acc, sm_ml, warp, lane, d0);
    if (warp == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const size_t o = ((size_t)i * n_q + kvh * G + g) * HD + d0;
#pragma unroll
            for (int d = 0; d < DPL; d++) {
                const float y = st.acc[g][d] / st.l[g];
                if (OUT_F32)
                    reinterpret_cast<float*>(out)[o + d] = y;
                else
                    reinterpret_cast<__half*>(out)[o + d] = __float2half_rn(y);
            }
        }
    }
}

struct PushSplitScale {
    uint32_t n_splits;
    float scale;
};

inline KvOperand linear_f16(const BufView& b, int n_kv, int hd)
{
    return KvOperand{b.ptr, nullptr, nullptr, 0, 1, b.bytes / ((size_t)n_kv * hd * 2)};
}
inline KvOperand linear_q8(const BufView& quants, const BufView& scales, int n_kv, int hd)
{
    return KvOperand{quants.ptr, (const __half*)scales.ptr, nullptr, 0, 1, quants.bytes / ((size_t)n_kv * hd)};
}

}  // namespace

// attn_decode_sliding / attn_decode_global / attn_decode_global_q8k and their d128 forms.
// bindings: q, k [, k_scales], v, part, step.  push {n_splits, scale}.  grid [n_kv, n_splits, m_q or 1].
template <int HD, int G, int KFMT, int VFMT, int STEP_SLOT>
int launch_decode_generic(const LaunchArgs& a)
{
    const PushSplitScale p = *(const PushSplitScale*)a.push;
    const int n_kv = (int)a.groups[0];
    const uint32_t m_q = a.groups[2] ? a.groups[2] : 1;
    if (n_kv <= 0 || p.n_splits == 0) return fail_validation(a, "decode: groups[0] (kv heads) and n_splits must be > 0");
    if (a.groups[1] != p.n_splits) return fail_validation(a, "decode: groups[1] must equal push.n_splits");
    int bi = 0;
    const BufView& q = a.b[bi++];
    KvOperand kop, vop;
    if (KFMT == FMT_Q8) {
        kop = linear_q8(a.b[bi], a.b[bi + 1], n_kv, HD);
        if (a.b[bi + 1].bytes / 2 < kop.rows * n_kv * (HD / 32)) return fail_validation(a, "decode: k_scales too short");
        bi += 2;
    } else {
        kop = linear_f16(a.b[bi++], n_kv, HD);
    }
    if (VFMT == FMT_Q8) {
        vop = linear_q8(a.b[bi], a.b[bi + 1], n_kv, HD);
        if (a.b[bi + 1].bytes / 2 < vop.rows * n_kv * (HD / 32)) return fail_validation(a, "decode: v_scales too short");
        bi += 2;
    } else {
        vop = linear_f16(a.b[bi++], n_kv, HD);
    }
    const int part_i = bi++, step_i = bi++;
    const size_t n_q = (size_t)n_kv * G;
    if (q.bytes < m_q * n_q * HD * 2) return fail_validation(a, "decode: q buffer too small");
    if (int r = need_bytes(a, part_i, m_q * n_q * p.n_splits * (HD + 2) * 4, "part")) return r;
    if (int r = need_bytes(a, step_i, 16, "step")) return r;
    decode_generic_kernel<HD, G, KFMT, VFMT><<<dim3(n_kv, p.n_splits, m_q), GEN_THREADS, 0, a.stream>>>(
        (const __half*)q.ptr, kop, vop, (float*)a.b[part_i].ptr, (const uint32_t*)a.b[step_i].ptr, STEP_SLOT, p.n_splits,
        p.scale, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_decode");
}
template int launch_decode_generic<256, 2, FMT_F16, FMT_F16, STEP_KV_LEN_SLIDING>(const LaunchArgs&);
template int launch_decode_generic<512, 8, FMT_F16, FMT_F16, STEP_KV_LEN_GLOBAL>(const LaunchArgs&);
template int launch_decode_generic<512, 8, FMT_Q8, FMT_F16, STEP_KV_LEN_GLOBAL>(const LaunchArgs&);
template int launch_decode_generic<128, 2, FMT_F16, FMT_F16, STEP_KV_LEN_SLIDING>(const LaunchArgs&);

struct PushDecodePaged {
    uint32_t n_splits;
    float scale;
    uint32_t page;
};

// The scalar statement of the paged Q8_0 decode (same bindings and push as the fast kernel):
// q, k_quants, k_scales, v_quants, v_scales, page_table, part, step.  push {n_splits, scale, page}.
int launch_decode_paged_q8kv_scalar_d128(const LaunchArgs& a)
{
    const PushDecodePaged p = *(const PushDecodePaged*)a.push;
    const int n_kv = (int)a.groups[0];
    const uint32_t m_q = a.groups[2] ? a.groups[2] : 1;
    if (n_kv <= 0 || p.n_splits == 0 || p.page == 0)
        return fail_validation(a, "decode_paged: kv heads, n_splits and page must be > 0");
    if (a.groups[1] != p.n_splits) return fail_validation(a, "decode_paged: groups[1] must equal push.n_splits");
    KvOperand kop = linear_q8(a.b[1], a.b[2], n_kv, 128), vop = linear_q8(a.b[3], a.b[4], n_kv, 128);
    if (a.b[2].bytes / 2 < kop.rows * n_kv * 4 || a.b[4].bytes / 2 < vop.rows * n_kv * 4)
        return fail_validation(a, "decode_paged: scales buffer too short for its quants buffer");
    kop.page_table = vop.page_table = (const uint32_t*)a.b[5].ptr;
    kop.table_len = vop.table_len = (uint32_t)(a.b[5].bytes / 4);
    kop.page = vop.page = p.page;
    const size_t n_q = (size_t)n_kv * 2;
    if (a.b[0].bytes < m_q * n_q * 128 * 2) return fail_validation(a, "decode_paged: q buffer too small");
    if (int r = need_bytes(a, 6, m_q * n_q * p.n_splits * 130 * 4, "part")) return r;
    if (int r = need_bytes(a, 7, 16, "step")) return r;
    decode_generic_kernel<128, 2, FMT_Q8, FMT_Q8><<<dim3(n_kv, p.n_splits, m_q), GEN_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, kop, vop, (float*)a.b[6].ptr, (const uint32_t*)a.b[7].ptr, STEP_KV_LEN_GLOBAL, p.n_splits,
        p.scale, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_decode_paged_q8kv_scalar_d128");
}

// attn_reduce_*: bindings part, out.  push {n_splits}.  grid [rows] (32 q heads in the reference).
template <int HD, int OUT_MODE>
int launch_reduce(const LaunchArgs& a)
{
    const uint32_t n_splits = *(const uint32_t*)a.push;
    const size_t rows = a.groups[0];
    if (rows == 0 || n_splits == 0 || n_splits > (uint32_t)REDUCE_MAX_SPLITS)
        return fail_validation(a, "attn_reduce: groups[0] (rows) must be > 0 and n_splits in 1..1024");
    if (int r = need_bytes(a, 0, rows * n_splits * (HD + 2) * 4, "part")) return r;
    const size_t out_bytes = OUT_MODE == 0 ? rows * HD * 2 : OUT_MODE == 1 ? rows * HD * 4 : rows * (HD + 2) * 4;
    if (int r = need_bytes(a, 1, out_bytes, "out")) return r;
    const cudaError_t e = launch_dependent(reduce_kernel<HD, OUT_MODE>, dim3((uint32_t)rows), dim3(HD / 2), 0, a.stream, (const float*)a.b[0].ptr,
                                           a.b[1].ptr, n_splits, 0);
    ++*a.launches;
    return check_cuda(a, e, "attn_reduce");
}
template int launch_reduce<256, 0>(const LaunchArgs&);
template int launch_reduce<512, 0>(const LaunchArgs&);
template int launch_reduce<128, 0>(const LaunchArgs&);
template int launch_reduce<128, 1>(const LaunchArgs&);
template int launch_reduce<128, 2>(const LaunchArgs&);

// attn_combine_ranks_d128: bindings gathered [n_ranks][rows][130] f32, out f32 [rows][128].
// push {n_ranks}.  grid [rows].  Ranks are merged in rank order, so every rank computes the same bits.
int launch_combine_ranks_d128(const LaunchArgs& a)
{
    const uint32_t n_ranks = *(const uint32_t*)a.push;
    const size_t rows = a.groups[0];
    if (rows == 0 || n_ranks == 0 || n_ranks > (uint32_t)REDUCE_MAX_SPLITS)
        return fail_validation(a, "attn_combine_ranks: rows must be > 0 and n_ranks in 1..1024");
    if (int r = need_bytes(a, 0, rows * n_ranks * 130 * 4, "gathered partials")) return r;
    if (int r = need_bytes(a, 1, rows * 128 * 4, "out")) return r;
    reduce_kernel<128, 1><<<(uint32_t)rows, 64, 0, a.stream>>>((const float*)a.b[0].ptr, a.b[1].ptr, n_ranks, 1);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_combine_ranks_d128");
}

// attn_prefill_sliding / _sliding_ring / _global and the d128 f32-output forms.
// TWO_RANGE: bindings q, k_ring, v_ring, k_chunk, v_chunk, out, step; else q, k, v, out, step.
// push {scale}.  grid [n_kv, M].
template <int HD, int G, int WINDOW, int RING, int TWO_RANGE, int OUT_F32>
int launch_prefill_generic(const LaunchArgs& a)
{
    const float scale = *(const float*)a.push;
    const int n_kv = (int)a.groups[0];
    const size_t m = a.groups[1];
    if (n_kv <= 0 || m == 0) return fail_validation(a, "attn_prefill: groups must be [kv heads, query tokens]");
    const size_t n_q = (size_t)n_kv * G;
    KvOperand kh = linear_f16(a.b[1], n_kv, HD), vh = linear_f16(a.b[2], n_kv, HD), kc{}, vc{};
    int bi = 3;
    if (TWO_RANGE) {
        kc = linear_f16(a.b[3], n_kv, HD);
        vc = linear_f16(a.b[4], n_kv, HD);
        bi = 5;
        if (kh.rows < (size_t)RING || vh.rows < (size_t)RING) return fail_validation(a, "attn_prefill: ring buffers too small");
        if (kc.rows < m || vc.rows < m) return fail_validation(a, "attn_prefill: chunk K/V hold fewer than M rows");
    }
    if (a.b[0].bytes < m * n_q * HD * 2) return fail_validation(a, "attn_prefill: q buffer too small");
    if (int r = need_bytes(a, bi, m * n_q * HD * (OUT_F32 ? 4 : 2), "out")) return r;
    if (int r = need_bytes(a, bi + 1, 16, "step")) return r;
    prefill_generic_kernel<HD, G, FMT_F16, FMT_F16, TWO_RANGE, OUT_F32><<<dim3(n_kv, (uint32_t)m), GEN_THREADS, 0, a.stream>>>(
        a.b[0].ptr, nullptr, kh, vh, kc, vc, a.b[bi].ptr, (const uint32_t*)a.b[bi + 1].ptr, WINDOW, RING, scale,
        a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_prefill");
}
template int launch_prefill_generic<256, 2, 1024, 0, 0, 0>(const LaunchArgs&);     // attn_prefill_sliding
template int launch_prefill_generic<256, 2, 1024, 1024, 1, 0>(const LaunchArgs&);  // attn_prefill_sliding_ring
template int launch_prefill_generic<512, 8, 0, 0, 0, 0>(const LaunchArgs&);        // attn_prefill_global
template int launch_prefill_generic<128, 2, 1024, 0, 0, 1>(const LaunchArgs&);     // attn_prefill_sliding_f32_d128
template int launch_prefill_generic<128, 2, 1024, 1024, 1, 1>(const LaunchArgs&);  // attn_prefill_sliding_ring_f32_d128
template int launch_prefill_generic<128, 2, 0, 0, 0, 1>(const LaunchArgs&);        // attn_prefill_global_f32_d128

struct PushScalePage {
    float scale;
    uint32_t page;
};

// Scalar statement of the paged Q8_0 prefill: q, k_quants, k_scales, v_quants, v_scales,
// page_table, out f32, step.  push {scale, page}.  grid [n_kv, M].  Global causal.
int launch_prefill_paged_q8kv_scalar_d128(const LaunchArgs& a)
{
    const PushScalePage p = *(const PushScalePage*)a.push;
    const int n_kv = (int)a.groups[0];
    const size_t m = a.groups[1];
    if (n_kv <= 0 || m == 0 || p.page == 0) return fail_validation(a, "prefill_paged: kv heads, M and page must be > 0");
    KvOperand kop = linear_q8(a.b[1], a.b[2], n_kv, 128), vop = linear_q8(a.b[3], a.b[4], n_kv, 128);
    if (a.b[2].bytes / 2 < kop.rows * n_kv * 4 || a.b[4].bytes / 2 < vop.rows * n_kv * 4)
        return fail_validation(a, "prefill_paged: scales buffer too short for its quants buffer");
    kop.page_table = vop.page_table = (const uint32_t*)a.b[5].ptr;
    kop.table_len = vop.table_len = (uint32_t)(a.b[5].bytes / 4);
    kop.page = vop.page = p.page;
    const size_t n_q = (size_t)n_kv * 2;
    if (a.b[0].bytes < m * n_q * 128 * 2) return fail_validation(a, "prefill_paged: q buffer too small");
    if (int r = need_bytes(a, 6, m * n_q * 128 * 4, "out")) return r;
    if (int r = need_bytes(a, 7, 16, "step")) return r;
    KvOperand none{};
    prefill_generic_kernel<128, 2, FMT_Q8, FMT_Q8, 0, 1><<<dim3(n_kv, (uint32_t)m), GEN_THREADS, 0, a.stream>>>(
        a.b[0].ptr, nullptr, kop, vop, none, none, a.b[6].ptr, (const uint32_t*)a.b[7].ptr, 0, 0, p.scale, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_prefill_paged_q8kv_scalar_d128");
}

// The reference's tiled global-prefill names (crates/sg-gpu/build.rs:2207-2287), all hd 512 / 4 kv heads /
// 8 query heads per kv head, out f16, push {scale}, grid [32 query heads, M / 16] (one workgroup per query
// head and 16-row tile, attn_prefill_global_flash_sp.wgsl:68-75).  They differ in what they bind:
//   VARIANT 0  attn_prefill_global_flash, attn_prefill_global_flash_sp: q f16, k f16, v f16, out, step
//   VARIANT 1  attn_prefill_global_flash_sp_q8: q f16, k_quants, k_scales, v_quants, v_scales, out, step
//   VARIANT 2  attn_prefill_global_flash_sp_iq: q_i8, q_scales, k_quants, k_scales, v f16, out, step
// Served by the streaming kernel on the dequantised values (the reference's own test compares the int8
// kernel with attention over the dequantised Q and K, tests/parity_attn.rs:689-768).  Rows past the last
// visible key are never read, so K/V need not be padded to a 64-key tile as the reference's callers do.
template <int VARIANT>
int launch_prefill_global_flash_ref(const LaunchArgs& a)
{
    constexpr int HD = 512, G = 8, N_KV = 4, M_Q = 16;
    const float scale = *(const float*)a.push;
    if (a.groups[0] != (uint32_t)(N_KV * G) || a.groups[1] == 0)
        return fail_validation(a, "attn_prefill_global_flash*: groups must be [32 query heads, M / 16]");
    const size_t m = (size_t)a.groups[1] * M_Q, n_q = (size_t)N_KV * G;
    KvOperand kop, vop, none{};
    const __half* q_scales = nullptr;
    int bi = 1;
    if (VARIANT == 2) {
        if (a.b[0].bytes < m * n_q * HD || a.b[1].bytes < m * n_q * (HD / 32) * 2)
            return fail_validation(a, "attn_prefill_global_flash_sp_iq: q_i8 / q_scales too small for M rows");
        q_scales = (const __half*)a.b[1].ptr;
        bi = 2;
    } else if (a.b[0].bytes < m * n_q * HD * 2) {
        return fail_validation(a, "attn_prefill_global_flash*: q buffer too small");
    }
    if (VARIANT == 0) {
        kop = linear_f16(a.b[bi], N_KV, HD);
        vop = linear_f16(a.b[bi + 1], N_KV, HD);
        bi += 2;
    } else {
        kop = linear_q8(a.b[bi], a.b[bi + 1], N_KV, HD);
        if (a.b[bi + 1].bytes / 2 < kop.rows * N_KV * (HD / 32)) return fail_validation(a, "attn_prefill_global_flash*: k_scales too short");
        bi += 2;
        if (VARIANT == 1) {
            vop = linear_q8(a.b[bi], a.b[bi + 1], N_KV, HD);
            if (a.b[bi + 1].bytes / 2 < vop.rows * N_KV * (HD / 32)) return fail_validation(a, "attn_prefill_global_flash*: v_scales too short");
            bi += 2;
        } else {
            vop = linear_f16(a.b[bi++], N_KV, HD);
        }
    }
    if (int r = need_bytes(a, bi, m * n_q * HD * 2, "out")) return r;
    if (int r = need_bytes(a, bi + 1, 16, "step")) return r;
    const dim3 grid(N_KV, (uint32_t)m);
    void* out = a.b[bi].ptr;
    const uint32_t* step = (const uint32_t*)a.b[bi + 1].ptr;
    if (VARIANT == 0)
        prefill_generic_kernel<HD, G, FMT_F16, FMT_F16, 0, 0><<<grid, GEN_THREADS, 0, a.stream>>>(a.b[0].ptr, nullptr, kop, vop, none, none, out,
                                                                                               step, 0, 0, scale, a.status);
    else if (VARIANT == 1)
        prefill_generic_kernel<HD, G, FMT_Q8_F16, FMT_Q8_F16, 0, 0><<<grid, GEN_THREADS, 0, a.stream>>>(a.b[0].ptr, nullptr, kop, vop, none, none,
                                                                                                     out, step, 0, 0, scale, a.status);
    else
        prefill_generic_kernel<HD, G, FMT_Q8, FMT_F16, 0, 0, FMT_Q8><<<grid, GEN_THREADS, 0, a.stream>>>(a.b[0].ptr, q_scales, kop, vop, none,
                                                                                                      none, out, step, 0, 0, scale, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_prefill_global_flash*");
}
template int launch_prefill_global_flash_ref<0>(const LaunchArgs&);
template int launch_prefill_global_flash_ref<1>(const LaunchArgs&);
template int launch_prefill_global_flash_ref<2>(const LaunchArgs&);

}  // namespace sgb
