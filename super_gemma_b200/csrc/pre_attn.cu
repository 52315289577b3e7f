// The steps between the QKV projections and the attention kernels: per-head RMS norm (QK-norm, weightless
// V-norm), rotate-half RoPE from a host-filled cos/sin table, and the quantise-and-append of K and V.
//
// Reference chain per layer (crates/sg-model/src/graph.rs:552-610): rmsnorm(q), rmsnorm(k), rmsnorm(v, ones),
// rope(q), rope(k), append(k), append(v) -- seven launches with an f16 round trip between every two.  Here:
//   rmsnorm_256/512[_plus1], rope_sliding_q/k, rope_global_q/k   the reference's names, bindings and grids
//       (crates/sg-gpu/shaders/rmsnorm.wgsl, rope.wgsl; build.rs:84-157)
//   attn_norm_rope_d128                       norm + rope of a [rows x 128] tensor in one pass
//   kv_norm_rope_append_paged_q8_d128         norm(k) + rope(k) + norm(v) + Q8_0 quantise + paged append
// The fused kernels round to f16 exactly where the chain stores f16 (after the norm, after the rotation), so
// they give the bits of their own unfused pieces.  All of it is HBM-bound: the head_dim-128 kernels give a row to 16
// consecutive lanes (16-byte accesses, partner dims and block maxima by shuffle), the reference-named ones a 32-value
// block to a thread; the row's sum of squares always goes through a fixed shuffle tree (deterministic).
//
// Arithmetic (f32): inv = 1/sqrt(sum(x^2)/n + 1e-6); y = f16(x * inv * w)  [w or 1 + w];
// rope pair i couples dims (i, i + n/2), live for i < rot_dims/2: lo' = f16(lo*c - hi*s), hi' = f16(hi*c + lo*s).
#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int PRE_THREADS = 256;
constexpr float RMS_EPS = 1e-6f;

__device__ __forceinline__ void load_f16x32(const __half* p, float (&x)[32])
{
    const uint4* v = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint4 u = __ldg(v + i);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            x[i * 8 + j * 2] = f.x;
            x[i * 8 + j * 2 + 1] = f.y;
        }
    }
}

__device__ __forceinline__ void pack_f16x32(const float (&x)[32], uint4 (&out)[4])
{
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 h = __floats2half2_rn(x[i * 8 + j * 2], x[i * 8 + j * 2 + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        out[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

// Sum of squares of a row spread over BPR consecutive lanes (one 32-value block each): in-thread sum in index
// order, then an xor butterfly, which gives every lane the same bits.
template <int BPR>
__device__ __forceinline__ float row_inv_rms(const float (&x)[32])
{
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) ss = fmaf(x[i], x[i], ss);
#pragma unroll
    for (int d = 1; d < BPR; d <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    return rsqrtf(ss / (float)(BPR * 32) + RMS_EPS);
}

// y = f16(x * inv * weight) for this thread's block; PLUS_ONE: weight = 1 + w (rmsnorm.wgsl:52-58); w == nullptr: 1.
template <bool PLUS_ONE>
__device__ __forceinline__ void apply_norm(float (&x)[32], float inv, const float* __restrict__ w)
{
#pragma unroll
    for (int i = 0; i < 32; i++) {
        float weight = 1.0f;
        if (w != nullptr) weight = PLUS_ONE ? 1.0f + __ldg(w + i) : __ldg(w + i);
        x[i] = round_f16(x[i] * inv * weight);
    }
}

// rmsnorm_<ROW_LEN>[_plus1]: x f16[rows x ROW_LEN], w f32[ROW_LEN], y f16.  grid [rows].
template <int BPR, bool PLUS_ONE>
__global__ void __launch_bounds__(PRE_THREADS) rmsnorm_kernel(const __half* __restrict__ x, const float* __restrict__ w,
                                                              __half* __restrict__ y, size_t n_blocks)
{
    const size_t blk = (size_t)blockIdx.x * PRE_THREADS + threadIdx.x;
    const bool live = blk < n_blocks;  // whole rows only, and BPR divides 32: a row never straddles a warp
    float v[32];
    if (live) {
        load_f16x32(x + blk * 32, v);
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = 0.0f;
    }
    const float inv = row_inv_rms<BPR>(v);
    if (!live) return;
    apply_norm<PLUS_ONE>(v, inv, w + (blk % BPR) * 32);
    uint4 out[4];
    pack_f16x32(v, out);
    uint4* o = reinterpret_cast<uint4*>(y + blk * 32);
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = out[i];
}

// rope_*: in place over rows [token x head x head_dim], one thread per (row, live pair) (rope.wgsl:36-52).
__global__ void __launch_bounds__(PRE_THREADS) rope_kernel(__half* __restrict__ xs, const float2* __restrict__ cos_sin,
                                                           uint32_t head_dim, uint32_t half_rot, uint32_t n_heads, size_t pairs_total)
{
    const size_t g = (size_t)blockIdx.x * PRE_THREADS + threadIdx.x;
    if (g >= pairs_total) return;
    const size_t row = g / half_rot;
    const uint32_t pair = (uint32_t)(g % half_rot);
    const size_t token = row / n_heads;
    const float2 cs = __ldg(cos_sin + token * half_rot + pair);
    __half* lo = xs + row * head_dim + pair;
    __half* hi = lo + head_dim / 2;
    const float a = __half2float(*lo), b = __half2float(*hi);
    *lo = __float2half_rn(__fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)));
    *hi = __float2half_rn(__fadd_rn(__fmul_rn(b, cs.x), __fmul_rn(a, cs.y)));
}

// One 8-dim piece of a 128-dim row after norm and rotation, as f16-exact floats.  The 16 threads of a row are
// consecutive lanes (two rows per warp, 16-byte accesses); thread `o` owns dims [8 o, 8 o + 8) and gets its
// rotation partner's normalised values (dims +-64, lane o ^ 8) by shuffle.  Every lane of the warp must call
// it (dead lanes with live = false), and half_rot must be the same for the whole warp.
template <bool PLUS_ONE>
__device__ __forceinline__ void norm_rope_oct_d128(const __half* __restrict__ row_ptr, const float* __restrict__ w,
                                                    const float2* __restrict__ cs_row, uint32_t half_rot, int o, bool live,
                                                    float (&v)[8])
{
    if (live) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(row_ptr + 8 * o));
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = 0.0f;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);  // fixed tree: every lane gets the same bits
    const float inv = rsqrtf(ss / 128.0f + RMS_EPS);
    float wv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) wv[i] = 1.0f;
    if (w != nullptr && live) {
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + 8 * o)), w1 = __ldg(reinterpret_cast<const float4*>(w + 8 * o) + 1);
        const float t[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) wv[i] = PLUS_ONE ? 1.0f + t[i] : t[i];
    }
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = round_f16(v[i] * inv * wv[i]);
    if (half_rot == 0) return;
    float other[8];
#pragma unroll
    for (int i = 0; i < 8; i++) other[i] = __shfl_xor_sync(0xffffffffu, v[i], 8);
    const uint32_t pair0 = (uint32_t)(o & 7) * 8;
    if (!live || pair0 >= half_rot) return;
    const float4* cp = reinterpret_cast<const float4*>(cs_row + pair0);  // (cos, sin) pairs; 16-byte aligned: half_rot % 8 == 0
#pragma unroll
    for (int j = 0; j < 4; j++) {  // half_rot is a multiple of 8 (checked on the host): all 8 pairs of a live piece rotate
        const float4 cs = __ldg(cp + j);
        const float c[2] = {cs.x, cs.z}, sn[2] = {cs.y, cs.w};
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int i = 2 * j + e;
            // low half: lo*c - hi*s with lo = own; high half: hi*c + lo*s with hi = own
            v[i] = (o < 8) ? round_f16(__fsub_rn(__fmul_rn(v[i], c[e]), __fmul_rn(other[i], sn[e])))
                           : round_f16(__fadd_rn(__fmul_rn(v[i], c[e]), __fmul_rn(other[i], sn[e])));
        }
    }
}

__device__ __forceinline__ uint4 pack_f16x8(const float (&v)[8])
{
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// attn_norm_rope_d128: x f16[rows x 128] (rows = tokens x n_heads), w f32[128], cos_sin f32[tokens x rot/2 x 2], y f16.
template <bool PLUS_ONE>
__global__ void __launch_bounds__(PRE_THREADS) norm_rope_d128_kernel(const __half* __restrict__ x, const float* __restrict__ w,
                                                                     const float2* __restrict__ cos_sin, __half* __restrict__ y,
                                                                     uint32_t n_heads, uint32_t half_rot, uint32_t rows)
{
    // 32-bit index arithmetic (the host checks rows * 16 < 2^32): 64-bit divisions would cost more than the rest
    const uint32_t g = blockIdx.x * PRE_THREADS + threadIdx.x;
    const uint32_t row = g >> 4;
    const int o = (int)(g & 15);
    const bool live = row < rows;
    float v[8];
    norm_rope_oct_d128<PLUS_ONE>(x + (size_t)row * 128, w, cos_sin + (size_t)(row / n_heads) * half_rot, half_rot, o, live, v);
    if (live) *reinterpret_cast<uint4*>(y + (size_t)row * 128 + 8 * o) = pack_f16x8(v);
}

// Q8_0 of the 32-value block that four consecutive lanes hold (8 values each): the arithmetic of
// kv_quant_q8.wgsl:38-57 (see kv_codec.cu); the block maximum by two shuffles.  All lanes of the warp call it.
__device__ __forceinline__ void quant_oct_f32(const float (&x)[8], __half& scale, uint2& packed)
{
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(x[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fmul_rn(amax, 1.0f / 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    scale = __float2half_rn(d);
    uint32_t p[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i++) p[i >> 2] |= (uint32_t)(__float2int_rn(__fmul_rn(x[i], id)) & 0xFF) << (8 * (i & 3));
    packed = make_uint2(p[0], p[1]);
}

// kv_norm_rope_append_paged_q8_d128: three warp-aligned segments of 16 threads per row: K rows (norm with k_w, rope),
// V rows (weightless norm), both landing Q8_0-quantised at row page_table[t / page] * page + t % page with
// t = step[0] + token; and, for qkv_norm_rope_append_paged_q8_d128, Q rows (norm with q_w, rope, f16 out): the
// whole pre-attention step of a layer in one launch.
template <bool PLUS_ONE>
__global__ void __launch_bounds__(PRE_THREADS)
    kv_norm_rope_append_kernel(const __half* __restrict__ q_raw, const float* __restrict__ q_w, __half* __restrict__ q_out,
                               uint32_t n_q, uint32_t q_rows,
                               const __half* __restrict__ k_raw, const __half* __restrict__ v_raw, const float* __restrict__ k_w,
                               const float2* __restrict__ cos_sin, __half* __restrict__ k_scales, int8_t* __restrict__ k_quants,
                               __half* __restrict__ v_scales, int8_t* __restrict__ v_quants, const uint32_t* __restrict__ page_table,
                               uint32_t table_len, uint32_t page, const uint32_t* __restrict__ step, uint32_t n_kv, uint32_t half_rot,
                               uint32_t kv_rows, size_t dst_rows, uint32_t* status)
{
    pdl_wait();  // the raw q, k, v rows come from earlier kernels of the stream
    pdl_launch_dependents();
    // 32-bit index arithmetic (the host checks the thread count < 2^32): 64-bit divisions would cost more than the rest
    const uint32_t g = blockIdx.x * PRE_THREADS + threadIdx.x;
    const uint32_t seg = (kv_rows * 16 + 31) / 32 * 32;  // threads per K or V segment: whole warps
    float v[8];
    if (g >= 2 * seg) {
        const uint32_t row = (g - 2 * seg) >> 4;
        const int o = (int)(g & 15);
        const bool live = row < q_rows;
        norm_rope_oct_d128<PLUS_ONE>(q_raw + (size_t)row * 128, q_w, cos_sin + (size_t)(row / n_q) * half_rot, half_rot, o, live, v);
        if (live) *reinterpret_cast<uint4*>(q_out + (size_t)row * 128 + 8 * o) = pack_f16x8(v);
        return;
    }
    const bool is_v = g >= seg;
    const uint32_t row = (is_v ? g - seg : g) >> 4;  // (token, kv head)
    const int o = (int)(g & 15);
    const bool live = row < kv_rows;
    const uint32_t token = row / n_kv, head = row - token * n_kv;
    norm_rope_oct_d128<PLUS_ONE>((is_v ? v_raw : k_raw) + (size_t)row * 128, is_v ? nullptr : k_w, cos_sin + (size_t)token * half_rot,
                                 is_v ? 0u : half_rot, o, live, v);
    __half s;
    uint2 packed;
    quant_oct_f32(v, s, packed);
    if (!live) return;
    const uint32_t t = __ldg(step + STEP_POS) + token;
    const uint32_t p = t / page;
    if (p >= table_len) {
        report_error(status, DEV_ERR_BOUNDS, 104, p, table_len);
        return;
    }
    const size_t dst_row = (size_t)__ldg(page_table + p) * page + (t - p * page);
    if (dst_row >= dst_rows) {
        report_error(status, DEV_ERR_BOUNDS, 105, (uint32_t)dst_row, (uint32_t)dst_rows);
        return;
    }
    const size_t drow = dst_row * n_kv + head;  // row of [128] quants / [4] scales
    if ((o & 3) == 0) (is_v ? v_scales : k_scales)[drow * 4 + (o >> 2)] = s;
    *reinterpret_cast<uint2*>((is_v ? v_quants : k_quants) + drow * 128 + 8 * o) = packed;
}

inline uint32_t grid_for(size_t n) { return (uint32_t)((n + PRE_THREADS - 1) / PRE_THREADS); }

struct PushNormRope {
    uint32_t n_heads, rot_dims, plus_one;
};
struct PushKvNormRope {
    uint32_t row_len, page, rot_dims, plus_one;
};
struct PushQkvNormRope {
    uint32_t n_q_heads, row_len, page, rot_dims, plus_one;
};

}  // namespace

template <int ROW_LEN, int PLUS_ONE>
int launch_rmsnorm(const LaunchArgs& a)
{
    static_assert(ROW_LEN % 32 == 0 && 32 % (ROW_LEN / 32) == 0, "a row is 1..32 blocks that divide a warp");
    if (a.b[0].bytes % (ROW_LEN * 2)) return fail_validation(a, "rmsnorm: x is not whole rows");
    if (int r = need_bytes(a, 1, ROW_LEN * 4, "w")) return r;
    if (int r = need_bytes(a, 2, a.b[0].bytes, "y")) return r;
    const size_t n_blocks = a.b[0].bytes / 64;
    if (n_blocks == 0) return 0;
    rmsnorm_kernel<ROW_LEN / 32, PLUS_ONE != 0><<<grid_for(n_blocks), PRE_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, (const float*)a.b[1].ptr, (__half*)a.b[2].ptr, n_blocks);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "rmsnorm");
}
template int launch_rmsnorm<256, 0>(const LaunchArgs&);
template int launch_rmsnorm<256, 1>(const LaunchArgs&);
template int launch_rmsnorm<512, 0>(const LaunchArgs&);
template int launch_rmsnorm<512, 1>(const LaunchArgs&);

template <int HEAD_DIM, int ROT_DIMS, int N_HEADS>
int launch_rope(const LaunchArgs& a)
{
    if (a.b[0].bytes % (HEAD_DIM * 2 * N_HEADS)) return fail_validation(a, "rope: xs is not whole tokens");
    const size_t rows = a.b[0].bytes / (HEAD_DIM * 2);
    const size_t pairs = rows * (ROT_DIMS / 2);
    if (int r = need_bytes(a, 1, rows / N_HEADS * (ROT_DIMS / 2) * 8, "cos_sin")) return r;
    if (pairs == 0) return 0;
    rope_kernel<<<grid_for(pairs), PRE_THREADS, 0, a.stream>>>((__half*)a.b[0].ptr, (const float2*)a.b[1].ptr, HEAD_DIM, ROT_DIMS / 2,
                                                                 N_HEADS, pairs);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "rope");
}
template int launch_rope<256, 256, 32>(const LaunchArgs&);
template int launch_rope<256, 256, 16>(const LaunchArgs&);
template int launch_rope<512, 128, 32>(const LaunchArgs&);
template int launch_rope<512, 128, 4>(const LaunchArgs&);

// attn_norm_rope_d128: x, w, cos_sin, y.  push {n_heads, rot_dims (0 = no rotation), plus_one}.
int launch_norm_rope_d128(const LaunchArgs& a)
{
    const PushNormRope p = *(const PushNormRope*)a.push;
    if (p.n_heads == 0 || p.rot_dims > 128 || p.rot_dims % 16) return fail_validation(a, "attn_norm_rope_d128: n_heads > 0, rot_dims a multiple of 16 up to 128");
    if (a.b[0].bytes % (256 * (size_t)p.n_heads)) return fail_validation(a, "attn_norm_rope_d128: x is not whole tokens of n_heads x 128");
    const size_t rows = a.b[0].bytes / 256;
    if (int r = need_bytes(a, 1, 128 * 4, "w")) return r;
    if (int r = need_bytes(a, 2, rows / p.n_heads * (p.rot_dims / 2) * 8, "cos_sin")) return r;
    if (int r = need_bytes(a, 3, a.b[0].bytes, "y")) return r;
    if (rows == 0) return 0;
    if (rows >= (1u << 27)) return fail_validation(a, "attn_norm_rope_d128: at most 2^27 rows per launch");
    if (reinterpret_cast<uintptr_t>(a.b[2].ptr) & 15) return fail_validation(a, "attn_norm_rope_d128: cos_sin must be 16-byte aligned");
    auto kern = p.plus_one ? norm_rope_d128_kernel<true> : norm_rope_d128_kernel<false>;
    kern<<<grid_for(rows * 16), PRE_THREADS, 0, a.stream>>>((const __half*)a.b[0].ptr, (const float*)a.b[1].ptr, (const float2*)a.b[2].ptr,
                                                           (__half*)a.b[3].ptr, p.n_heads, p.rot_dims / 2, (uint32_t)rows);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_norm_rope_d128");
}

// kv_norm_rope_append_paged_q8_d128: k_raw, v_raw f16[n x row_len], k_w f32[128], cos_sin, k_scales, k_quants,
// v_scales, v_quants, page_table, step.  push {row_len, page, rot_dims, plus_one}.
int launch_kv_norm_rope_append_paged_q8_d128(const LaunchArgs& a)
{
    const PushKvNormRope p = *(const PushKvNormRope*)a.push;
    if (p.row_len == 0 || p.row_len % 128 || p.page == 0 || p.rot_dims > 128 || p.rot_dims % 16)
        return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: row_len = n_kv_heads*128, page > 0, rot_dims a multiple of 16 up to 128");
    if (a.b[0].bytes % (p.row_len * 2) || a.b[1].bytes != a.b[0].bytes)
        return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: k_raw and v_raw must be the same whole rows");
    const size_t tokens = a.b[0].bytes / (p.row_len * 2);
    if (int r = need_bytes(a, 2, 128 * 4, "k_w")) return r;
    if (int r = need_bytes(a, 3, tokens * (p.rot_dims / 2) * 8, "cos_sin")) return r;
    if (int r = need_bytes(a, 9, 16, "step")) return r;
    const size_t dst_rows = a.b[5].bytes / p.row_len;
    if (a.b[7].bytes / p.row_len != dst_rows) return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: K and V pools differ in rows");
    if (a.b[4].bytes / 2 < dst_rows * (p.row_len / 32) || a.b[6].bytes / 2 < dst_rows * (p.row_len / 32))
        return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: scales buffer too short for the quants buffer");
    const size_t kv_rows = a.b[0].bytes / 256;
    if (kv_rows == 0) return 0;
    if (kv_rows >= (1u << 26)) return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: at most 2^26 (token, head) rows per launch");
    if (reinterpret_cast<uintptr_t>(a.b[3].ptr) & 15) return fail_validation(a, "kv_norm_rope_append_paged_q8_d128: cos_sin must be 16-byte aligned");
    const size_t seg = (kv_rows * 16 + 31) / 32 * 32;
    auto kern = p.plus_one ? kv_norm_rope_append_kernel<true> : kv_norm_rope_append_kernel<false>;
    const cudaError_t e = launch_dependent(kern, dim3(grid_for(2 * seg)), dim3(PRE_THREADS), 0, a.stream,
        nullptr, nullptr, nullptr, 1u, 0u,
        (const __half*)a.b[0].ptr, (const __half*)a.b[1].ptr, (const float*)a.b[2].ptr, (const float2*)a.b[3].ptr, (__half*)a.b[4].ptr,
        (int8_t*)a.b[5].ptr, (__half*)a.b[6].ptr, (int8_t*)a.b[7].ptr, (const uint32_t*)a.b[8].ptr, (uint32_t)(a.b[8].bytes / 4), p.page,
        (const uint32_t*)a.b[9].ptr, p.row_len / 128, p.rot_dims / 2, (uint32_t)kv_rows, dst_rows, a.status);
    ++*a.launches;
    return check_cuda(a, e, "kv_norm_rope_append_paged_q8_d128");
}

// qkv_norm_rope_append_paged_q8_d128: q_raw f16[n x n_q x128], q_w f32[128], q_out f16, then the ten bindings of
// kv_norm_rope_append_paged_q8_d128.  push {n_q_heads, row_len, page, rot_dims, plus_one}.
int launch_qkv_norm_rope_append_paged_q8_d128(const LaunchArgs& a)
{
    const PushQkvNormRope p = *(const PushQkvNormRope*)a.push;
    if (p.n_q_heads == 0 || p.row_len == 0 || p.row_len % 128 || p.page == 0 || p.rot_dims > 128 || p.rot_dims % 16)
        return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: n_q_heads > 0, row_len = n_kv_heads*128, page > 0, rot_dims a multiple of 16 up to 128");
    const BufView* kv = a.b + 3;
    if (kv[0].bytes % (p.row_len * 2) || kv[1].bytes != kv[0].bytes)
        return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: k_raw and v_raw must be the same whole rows");
    const size_t tokens = kv[0].bytes / (p.row_len * 2);
    if (a.b[0].bytes != tokens * p.n_q_heads * 256) return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: q_raw must hold the same tokens");
    if (int r = need_bytes(a, 1, 128 * 4, "q_w")) return r;
    if (int r = need_bytes(a, 2, a.b[0].bytes, "q_out")) return r;
    if (int r = need_bytes(a, 5, 128 * 4, "k_w")) return r;
    if (int r = need_bytes(a, 6, tokens * (p.rot_dims / 2) * 8, "cos_sin")) return r;
    if (int r = need_bytes(a, 12, 16, "step")) return r;
    const size_t dst_rows = kv[5].bytes / p.row_len;
    if (kv[7].bytes / p.row_len != dst_rows) return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: K and V pools differ in rows");
    if (kv[4].bytes / 2 < dst_rows * (p.row_len / 32) || kv[6].bytes / 2 < dst_rows * (p.row_len / 32))
        return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: scales buffer too short for the quants buffer");
    const size_t kv_rows = kv[0].bytes / 256, q_rows = a.b[0].bytes / 256;
    if (kv_rows == 0) return 0;
    if (kv_rows >= (1u << 26) || q_rows >= (1u << 26))
        return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: at most 2^26 (token, head) rows of q and of k per launch");
    if (reinterpret_cast<uintptr_t>(kv[3].ptr) & 15) return fail_validation(a, "qkv_norm_rope_append_paged_q8_d128: cos_sin must be 16-byte aligned");
    const size_t seg = (kv_rows * 16 + 31) / 32 * 32;
    auto kern = p.plus_one ? kv_norm_rope_append_kernel<true> : kv_norm_rope_append_kernel<false>;
    const cudaError_t e = launch_dependent(kern, dim3(grid_for(2 * seg + q_rows * 16)), dim3(PRE_THREADS), 0, a.stream,
        (const __half*)a.b[0].ptr, (const float*)a.b[1].ptr, (__half*)a.b[2].ptr, p.n_q_heads, (uint32_t)q_rows, (const __half*)kv[0].ptr,
        (const __half*)kv[1].ptr, (const float*)kv[2].ptr, (const float2*)kv[3].ptr, (__half*)kv[4].ptr, (int8_t*)kv[5].ptr,
        (__half*)kv[6].ptr, (int8_t*)kv[7].ptr, (const uint32_t*)kv[8].ptr, (uint32_t)(kv[8].bytes / 4), p.page,
        (const uint32_t*)kv[9].ptr, p.row_len / 128, p.rot_dims / 2, (uint32_t)kv_rows, dst_rows, a.status);
    ++*a.launches;
    return check_cuda(a, e, "qkv_norm_rope_append_paged_q8_d128");
}

}  // namespace sgb
