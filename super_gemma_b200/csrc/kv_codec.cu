// Q8_0 codec and KV placement kernels.
//
// Format (crates/sg-gpu/shaders/kv_quant_q8.wgsl:1-18): structure of arrays -- one f16 scale per
// 32 consecutive values of a row, and the int8 quants in row order.  Arithmetic that decides bits:
//   d  = amax * (1/127)      (an f32 MULTIPLY, kv_quant_q8.wgsl:42)
//   scale = RTNE f16(d);  id = d > 0 ? 1/d : 0;  q = round_half_even(x * id)
//   dequant: f16(f32(scale) * f32(q))            (kv_dequant_q8.wgsl:26)
// All of them are HBM-bound byte shuffles: 16-byte accesses, one block of 32 values per thread.
#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int CODEC_THREADS = 256;

// Quantise one 32-value block held as 4 x uint4 of f16; returns the scale and 8 packed words.
__device__ __forceinline__ void quant_block(const uint4 (&in)[4], __half& scale, uint32_t (&packed)[8])
{
    float x[32];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2* h = reinterpret_cast<const __half2*>(&in[i]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = __half22float2(h[j]);
            x[i * 8 + j * 2] = f.x;
            x[i * 8 + j * 2 + 1] = f.y;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
    const float d = __fmul_rn(amax, 1.0f / 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    scale = __float2half_rn(d);
#pragma unroll
    for (int w = 0; w < 8; w++) {
        uint32_t p = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int q = __float2int_rn(__fmul_rn(x[w * 4 + b], id));
            p |= (uint32_t)(q & 0xFF) << (8 * b);
        }
        packed[w] = p;
    }
}

__device__ __forceinline__ void load_block(const __half* src, size_t blk, uint4 (&in)[4])
{
    const uint4* p = reinterpret_cast<const uint4*>(src + blk * 32);
#pragma unroll
    for (int i = 0; i < 4; i++) in[i] = __ldg(p + i);
}

__device__ __forceinline__ void store_quants(int8_t* quants, size_t blk, const uint32_t (&packed)[8])
{
    uint4* o = reinterpret_cast<uint4*>(quants + blk * 32);
    o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// kv_quant_q8 (crates/sg-gpu/shaders/kv_quant_q8.wgsl:24-57).
__global__ void __launch_bounds__(CODEC_THREADS) kv_quant_q8_kernel(const __half* __restrict__ src,
                                                                    __half* __restrict__ scales,
                                                                    int8_t* __restrict__ quants, size_t n_blocks)
{
    const size_t blk = (size_t)blockIdx.x * CODEC_THREADS + threadIdx.x;
    if (blk >= n_blocks) return;
    uint4 in[4];
    load_block(src, blk, in);
    __half s;
    uint32_t packed[8];
    quant_block(in, s, packed);
    scales[blk] = s;
    store_quants(quants, blk, packed);
}

// kv_dequant_q8 (crates/sg-gpu/shaders/kv_dequant_q8.wgsl:9-29): one thread per 16 values.
__global__ void __launch_bounds__(CODEC_THREADS) kv_dequant_q8_kernel(const __half* __restrict__ scales,
                                                                      const int8_t* __restrict__ quants,
                                                                      __half* __restrict__ dst, size_t n_halfblocks)
{
    const size_t hb = (size_t)blockIdx.x * CODEC_THREADS + threadIdx.x;
    if (hb >= n_halfblocks) return;
    const float d = __half2float(scales[hb >> 1]);
    const uint4 qw = __ldg(reinterpret_cast<const uint4*>(quants) + hb);
    const uint32_t w[4] = {qw.x, qw.y, qw.z, qw.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float f0 = __fmul_rn(d, (float)(int8_t)(w[i] & 0xFF));
        const float f1 = __fmul_rn(d, (float)(int8_t)((w[i] >> 8) & 0xFF));
        const float f2 = __fmul_rn(d, (float)(int8_t)((w[i] >> 16) & 0xFF));
        const float f3 = __fmul_rn(d, (float)(int8_t)(w[i] >> 24));
        o[2 * i] = pack_half2(f0, f1);
        o[2 * i + 1] = pack_half2(f2, f3);
    }
    uint4* out = reinterpret_cast<uint4*>(dst) + hb * 2;
    out[0] = make_uint4(o[0], o[1], o[2], o[3]);
    out[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// kv_append (crates/sg-gpu/shaders/kv_append.wgsl:15-37): rows of ROW_LEN f16, slot from step[0].
template <int ROW_LEN, int RING>
__global__ void __launch_bounds__(CODEC_THREADS) kv_append_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                  const uint32_t* __restrict__ step, size_t n_vec,
                                                                  size_t dst_rows, uint32_t* status)
{
    constexpr int VEC_PER_ROW = ROW_LEN / 8;
    const size_t i = (size_t)blockIdx.x * CODEC_THREADS + threadIdx.x;
    if (i >= n_vec) return;
    const size_t token = i / VEC_PER_ROW, j = i % VEC_PER_ROW;
    size_t slot = (size_t)step[STEP_POS] + token;
    if (RING > 0) slot %= RING;
    if (slot >= dst_rows) {
        report_error(status, DEV_ERR_BOUNDS, 101, (uint32_t)slot, (uint32_t)dst_rows);
        return;
    }
    dst[slot * VEC_PER_ROW + j] = __ldg(src + i);
}

// kv_append_global_q8 (crates/sg-gpu/shaders/kv_append_global_q8.wgsl:19-60), plus the page-table
// row mapping when page_table != nullptr: row = page_table[t / page] * page + t % page.
__global__ void __launch_bounds__(CODEC_THREADS) kv_append_q8_kernel(const __half* __restrict__ src,
                                                                     __half* __restrict__ scales,
                                                                     int8_t* __restrict__ quants,
                                                                     const uint32_t* __restrict__ page_table,
                                                                     uint32_t table_len, uint32_t page,
                                                                     const uint32_t* __restrict__ step,
                                                                     uint32_t blocks_per_row, size_t n_blocks,
                                                                     size_t dst_rows, uint32_t* status)
{
    const size_t blk = (size_t)blockIdx.x * CODEC_THREADS + threadIdx.x;
    if (blk >= n_blocks) return;
    const size_t token = blk / blocks_per_row, local = blk % blocks_per_row;
    size_t t = (size_t)step[STEP_POS] + token;
    size_t row = t;
    if (page_table != nullptr) {
        const size_t p = t / page;
        if (p >= table_len) {
            report_error(status, DEV_ERR_BOUNDS, 102, (uint32_t)p, table_len);
            return;
        }
        row = (size_t)page_table[p] * page + t % page;
    }
    if (row >= dst_rows) {
        report_error(status, DEV_ERR_BOUNDS, 103, (uint32_t)row, (uint32_t)dst_rows);
        return;
    }
    uint4 in[4];
    load_block(src, blk, in);
    __half s;
    uint32_t packed[8];
    quant_block(in, s, packed);
    const size_t dblk = row * blocks_per_row + local;
    scales[dblk] = s;
    store_quants(quants, dblk, packed);
}

// Gather + dequantise the first kv_len logical tokens of a paged Q8_0 pool into linear f16 rows (and zero
// the rows up to the next multiple of 64):
// dst[t][j] = f16(scale * q) read at row page_table[t / page] * page + t % page.  The dequantised
// value is the one attn_prefill_global_flash_sp_q8.wgsl:100-104 builds in its LDS slab.
__global__ void __launch_bounds__(CODEC_THREADS) kv_dequant_paged_kernel(const __half* __restrict__ scales,
                                                                         const int8_t* __restrict__ quants,
                                                                         const uint32_t* __restrict__ page_table,
                                                                         uint32_t table_len, uint32_t page,
                                                                         __half* __restrict__ dst,
                                                                         const uint32_t* __restrict__ step,
                                                                         uint32_t row_len, size_t dst_rows,
                                                                         size_t src_rows, uint32_t* status)
{
    const uint32_t hb_per_row = row_len / 16;
    const size_t kv_len = step[STEP_KV_LEN_GLOBAL];
    // The flash kernel reads whole 64-key tiles and masks what lies past kv_len; a masked key weighs 0, but
    // 0 times a stale inf or NaN would not be 0, so the rest of the last tile is zeroed here.
    const size_t padded = (kv_len + 63) / 64 * 64;
    const size_t n_rows = padded < dst_rows ? padded : dst_rows;
    for (size_t i = (size_t)blockIdx.x * CODEC_THREADS + threadIdx.x; i < n_rows * hb_per_row;
         i += (size_t)gridDim.x * CODEC_THREADS) {
        const size_t t = i / hb_per_row, hb = i % hb_per_row;
        if (t >= kv_len) {
            uint4* out = reinterpret_cast<uint4*>(dst + t * row_len) + hb * 2;
            out[0] = out[1] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const size_t p = t / page;
        if (p >= table_len) {
            report_error(status, DEV_ERR_BOUNDS, 104, (uint32_t)p, table_len);
            return;
        }
        const size_t row = (size_t)page_table[p] * page + t % page;
        if (row >= src_rows) {
            report_error(status, DEV_ERR_BOUNDS, 105, (uint32_t)row, (uint32_t)src_rows);
            return;
        }
        const float d = __half2float(scales[row * (row_len / 32) + (hb >> 1)]);
        const uint4 qw = __ldg(reinterpret_cast<const uint4*>(quants + row * row_len) + hb);
        const uint32_t w[4] = {qw.x, qw.y, qw.z, qw.w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float f0 = __fmul_rn(d, (float)(int8_t)(w[k] & 0xFF));
            const float f1 = __fmul_rn(d, (float)(int8_t)((w[k] >> 8) & 0xFF));
            const float f2 = __fmul_rn(d, (float)(int8_t)((w[k] >> 16) & 0xFF));
            const float f3 = __fmul_rn(d, (float)(int8_t)(w[k] >> 24));
            o[2 * k] = pack_half2(f0, f1);
            o[2 * k + 1] = pack_half2(f2, f3);
        }
        uint4* out = reinterpret_cast<uint4*>(dst + t * row_len) + hb * 2;
        out[0] = make_uint4(o[0], o[1], o[2], o[3]);
        out[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

inline uint32_t blocks_for(size_t n, int per_block) { return (uint32_t)((n + per_block - 1) / per_block); }

}  // namespace

// bindings: src f16, scales f16, quants i8.  Covers src.len / 32 blocks (arrayLength semantics).
int launch_kv_quant_q8(const LaunchArgs& a)
{
    const size_t n_blocks = a.b[0].bytes / 2 / 32;
    if (a.b[0].bytes % 64) return fail_validation(a, "kv_quant_q8: src length must be a multiple of 32 values");
    if (int r = need_bytes(a, 1, n_blocks * 2, "scales")) return r;
    if (int r = need_bytes(a, 2, n_blocks * 32, "quants")) return r;
    if (n_blocks == 0) return 0;
    kv_quant_q8_kernel<<<blocks_for(n_blocks, CODEC_THREADS), CODEC_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, (__half*)a.b[1].ptr, (int8_t*)a.b[2].ptr, n_blocks);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_quant_q8");
}

// bindings: scales f16, quants i8, dst f16.  Covers dst.len / 32 blocks.
int launch_kv_dequant_q8(const LaunchArgs& a)
{
    const size_t n_blocks = a.b[2].bytes / 2 / 32;
    if (a.b[2].bytes % 64) return fail_validation(a, "kv_dequant_q8: dst length must be a multiple of 32 values");
    if (int r = need_bytes(a, 0, n_blocks * 2, "scales")) return r;
    if (int r = need_bytes(a, 1, n_blocks * 32, "quants")) return r;
    if (n_blocks == 0) return 0;
    kv_dequant_q8_kernel<<<blocks_for(n_blocks * 2, CODEC_THREADS), CODEC_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, (const int8_t*)a.b[1].ptr, (__half*)a.b[2].ptr, n_blocks * 2);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_dequant_q8");
}

// bindings: src f16 [n x ROW_LEN], dst f16 [slots x ROW_LEN], step.
template <int ROW_LEN, int RING>
int launch_kv_append(const LaunchArgs& a)
{
    static_assert(ROW_LEN % 8 == 0, "rows are copied in 16-byte pieces");
    if (a.b[0].bytes % (ROW_LEN * 2)) return fail_validation(a, "kv_append: src is not a whole number of rows");
    if (int r = need_bytes(a, 2, 16, "step")) return r;
    const size_t n_vec = a.b[0].bytes / 16;
    const size_t dst_rows = a.b[1].bytes / (ROW_LEN * 2);
    if (RING > 0 && dst_rows < (size_t)RING) return fail_validation(a, "kv_append: ring buffer smaller than the ring");
    if (n_vec == 0) return 0;
    kv_append_kernel<ROW_LEN, RING><<<blocks_for(n_vec, CODEC_THREADS), CODEC_THREADS, 0, a.stream>>>(
        (const uint4*)a.b[0].ptr, (uint4*)a.b[1].ptr, (const uint32_t*)a.b[2].ptr, n_vec, dst_rows, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_append");
}
template int launch_kv_append<4096, 1024>(const LaunchArgs&);  // kv_append_sliding (16 kv heads x 256)
template int launch_kv_append<2048, 0>(const LaunchArgs&);     // kv_append_global  (4 kv heads x 512)
template int launch_kv_append<2048, 1024>(const LaunchArgs&);  // kv_append_sliding_d128 (16 kv heads x 128)

// bindings: src f16 [n x ROW_LEN], scales f16, quants i8, step.
template <int ROW_LEN>
int launch_kv_append_global_q8(const LaunchArgs& a)
{
    if (a.b[0].bytes % (ROW_LEN * 2)) return fail_validation(a, "kv_append_global_q8: src is not whole rows");
    if (int r = need_bytes(a, 3, 16, "step")) return r;
    const size_t n_blocks = a.b[0].bytes / 64;
    const size_t dst_rows = a.b[2].bytes / ROW_LEN;
    if (a.b[1].bytes / 2 < dst_rows * (ROW_LEN / 32))
        return fail_validation(a, "kv_append_global_q8: scales buffer shorter than the quants buffer implies");
    if (n_blocks == 0) return 0;
    kv_append_q8_kernel<<<blocks_for(n_blocks, CODEC_THREADS), CODEC_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, (__half*)a.b[1].ptr, (int8_t*)a.b[2].ptr, nullptr, 0, 1, (const uint32_t*)a.b[3].ptr,
        ROW_LEN / 32, n_blocks, dst_rows, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_append_global_q8");
}
template int launch_kv_append_global_q8<2048>(const LaunchArgs&);

struct PushRowPage {
    uint32_t row_len;
    uint32_t page;
};

// bindings: src f16 [n x row_len], scales f16, quants i8, page_table u32, step.  push {row_len, page}.
int launch_kv_append_paged_q8_d128(const LaunchArgs& a)
{
    const PushRowPage p = *(const PushRowPage*)a.push;
    if (p.row_len == 0 || p.row_len % 128 || p.page == 0)
        return fail_validation(a, "kv_append_paged_q8_d128: row_len must be n_kv_heads*128 and page > 0");
    if (a.b[0].bytes % (p.row_len * 2)) return fail_validation(a, "kv_append_paged_q8_d128: src is not whole rows");
    if (int r = need_bytes(a, 4, 16, "step")) return r;
    const size_t n_blocks = a.b[0].bytes / 64;
    const size_t dst_rows = a.b[2].bytes / p.row_len;
    if (a.b[1].bytes / 2 < dst_rows * (p.row_len / 32))
        return fail_validation(a, "kv_append_paged_q8_d128: scales buffer too short for the quants buffer");
    if (n_blocks == 0) return 0;
    kv_append_q8_kernel<<<blocks_for(n_blocks, CODEC_THREADS), CODEC_THREADS, 0, a.stream>>>(
        (const __half*)a.b[0].ptr, (__half*)a.b[1].ptr, (int8_t*)a.b[2].ptr, (const uint32_t*)a.b[3].ptr,
        (uint32_t)(a.b[3].bytes / 4), p.page, (const uint32_t*)a.b[4].ptr, p.row_len / 32, n_blocks, dst_rows, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_append_paged_q8_d128");
}

// Shared with the paged flash prefill launcher.
int run_kv_dequant_paged(const LaunchArgs& a, const BufView& scales, const BufView& quants, const BufView& table,
                         const BufView& dst, const BufView& step, uint32_t row_len, uint32_t page)
{
    const size_t dst_rows = dst.bytes / ((size_t)row_len * 2);
    const size_t src_rows = quants.bytes / row_len;
    if (scales.bytes / 2 < src_rows * (row_len / 32))
        return fail_validation(a, "kv_dequant_paged: scales buffer too short for the quants buffer");
    if (dst_rows == 0) return 0;
    size_t want = (dst_rows * (row_len / 16) + CODEC_THREADS - 1) / CODEC_THREADS;
    const uint32_t grid = (uint32_t)(want < (size_t)a.sm_count * 16 ? want : (size_t)a.sm_count * 16);
    kv_dequant_paged_kernel<<<grid, CODEC_THREADS, 0, a.stream>>>(
        (const __half*)scales.ptr, (const int8_t*)quants.ptr, (const uint32_t*)table.ptr, (uint32_t)(table.bytes / 4), page,
        (__half*)dst.ptr, (const uint32_t*)step.ptr, row_len, dst_rows, src_rows, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "kv_dequant_paged");
}

// bindings: scales f16, quants i8, page_table u32, dst f16 [rows x row_len], step.  push {row_len, page}.
// Writes the first min(step.kv_len_global, dst rows) logical tokens.
int launch_kv_dequant_paged_q8_d128(const LaunchArgs& a)
{
    const PushRowPage p = *(const PushRowPage*)a.push;
    if (p.row_len == 0 || p.row_len % 128 || p.page == 0)
        return fail_validation(a, "kv_dequant_paged_q8_d128: row_len must be n_kv_heads*128 and page > 0");
    if (int r = need_bytes(a, 4, 16, "step")) return r;
    return run_kv_dequant_paged(a, a.b[0], a.b[1], a.b[2], a.b[3], a.b[4], p.row_len, p.page);
}

}  // namespace sgb
