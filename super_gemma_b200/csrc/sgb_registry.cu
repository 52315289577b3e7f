// The kernel registry: names, binding counts, push sizes and grid meaning.
//
// Reference-shaped entries keep the reference's registry name, binding order, push layout and grid
// (crates/sg-gpu/build.rs: the VARIANTS entries at :253-437) so a caller written against sg-gpu
// binds them unchanged.  Entries for the 32 q / 16 kv / head_dim 128 shapes and for inputs the
// reference kernels do not take (page table, Q8_0 V, f32 output) get NEW names: an existing
// binding list never changes meaning.  For those, the number of kv heads is groups[0], so a rank
// that owns a slice of the heads dispatches the same kernel with a smaller grid.
#include "sgb_kernels.h"

namespace sgb {

namespace {

enum : int { FMT_F16 = 0, FMT_Q8 = 1 };
enum : int { SLOT_SLIDING = 1, SLOT_GLOBAL = 2 };

const KernelEntry REGISTRY[] = {
    // ---- reference names (crates/sg-gpu/build.rs) -----------------------------------------------------
    {"attn_decode_sliding", {64, 1, 1}, 5, 8,
     "q f16[32x256], k_ring f16[slot x16x256], v_ring, part f32[32 x n_splits x 258], step | push {n_splits u32, scale f32} | "
     "grid [16 kv heads, n_splits]; kv_len = step[1]",
     launch_decode_generic<256, 2, FMT_F16, FMT_F16, SLOT_SLIDING>},
    {"attn_decode_global", {64, 1, 1}, 5, 8,
     "q f16[32x512], k f16[token x4x512], v, part f32[32 x n_splits x 514], step | push {n_splits, scale} | "
     "grid [4 kv heads, n_splits]; kv_len = step[2]",
     launch_decode_generic<512, 8, FMT_F16, FMT_F16, SLOT_GLOBAL>},
    {"attn_decode_global_q8k", {64, 1, 1}, 6, 8,
     "q f16[32x512], k_quants i8[token x4x512], k_scales f16[token x4x16], v f16, part f32[32 x n_splits x 514], step | "
     "push {n_splits, scale} | grid [4 kv heads, n_splits]; kv_len = step[2]",
     launch_decode_generic<512, 8, FMT_Q8, FMT_F16, SLOT_GLOBAL>},
    {"attn_reduce_d256", {64, 1, 1}, 2, 4, "part f32[rows x n_splits x 258], out f16[rows x 256] | push {n_splits} | grid [rows]",
     launch_reduce<256, 0>},
    {"attn_reduce_d512", {64, 1, 1}, 2, 4, "part f32[rows x n_splits x 514], out f16[rows x 512] | push {n_splits} | grid [rows]",
     launch_reduce<512, 0>},
    {"attn_prefill_sliding", {64, 1, 1}, 5, 4,
     "q f16[M x32x256], k f16[token x16x256], v, out f16[M x32x256], step | push {scale} | grid [16, M]; window 1024; q0 = step[3]",
     launch_prefill_generic<256, 2, 1024, 0, 0, 0>},
    {"attn_prefill_sliding_ring", {64, 1, 1}, 7, 4,
     "q, k_ring f16[1024x16x256], v_ring, k_chunk f16[M x16x256], v_chunk, out f16, step | push {scale} | grid [16, M]; "
     "history at slot pos % 1024 (pre-append ring), then the chunk's own rows",
     launch_prefill_generic<256, 2, 1024, 1024, 1, 0>},
    {"attn_prefill_global", {64, 1, 1}, 5, 4,
     "q f16[M x32x512], k f16[token x4x512], v, out f16, step | push {scale} | grid [4, M]; causal [0, q0+i]",
     launch_prefill_generic<512, 8, 0, 0, 0, 0>},
    // The tiled global-prefill variants (build.rs:2207-2287): grid [32 query heads, M / 16], K/V padded to a 64-key tile
    // by the reference's callers (not required here).  sg-model dispatches ..._flash_sp_iq for every global prefill layer
    // (crates/sg-model/src/graph.rs:1210-1223).
    {"attn_prefill_global_flash", {64, 1, 1}, 5, 4,
     "q f16[M x32x512], k f16[token x4x512], v, out f16[M x32x512], step | push {scale} | grid [32, M/16]; causal [0, q0+i]",
     launch_prefill_global_flash_ref<0>},
    {"attn_prefill_global_flash_sp", {64, 1, 1}, 5, 4,
     "q f16[M x32x512], k f16[token x4x512], v, out f16[M x32x512], step | push {scale} | grid [32, M/16]; causal [0, q0+i]",
     launch_prefill_global_flash_ref<0>},
    {"attn_prefill_global_flash_sp_q8", {64, 1, 1}, 7, 4,
     "q f16[M x32x512], k_quants i8[token x4x512], k_scales f16[token x4x16], v_quants, v_scales, out f16, step | push {scale} | "
     "grid [32, M/16]; K and V enter as f16(scale*q)",
     launch_prefill_global_flash_ref<1>},
    {"attn_prefill_global_flash_sp_iq", {64, 1, 1}, 7, 4,
     "q_i8 i8[M x32x512], q_scales f16[M x32x16], k_quants i8[token x4x512], k_scales f16[token x4x16], v f16[token x4x512], out f16, step | "
     "push {scale} | grid [32, M/16]; scores from the exact products f32(scale)*f32(q) of Q and K",
     launch_prefill_global_flash_ref<2>},
    {"kv_append_sliding", {256, 1, 1}, 3, 0, "src f16[n x4096], dst f16[1024 x4096], step | grid covers src; slot = (step[0]+token) % 1024",
     launch_kv_append<4096, 1024>},
    {"kv_append_global", {256, 1, 1}, 3, 0, "src f16[n x2048], dst f16[slots x2048], step | slot = step[0]+token",
     launch_kv_append<2048, 0>},
    {"kv_append_global_q8", {256, 1, 1}, 4, 0, "src f16[n x2048], scales f16[slots x64], quants i8[slots x2048], step | slot = step[0]+token",
     launch_kv_append_global_q8<2048>},
    {"kv_quant_q8", {256, 1, 1}, 3, 0, "src f16[n], scales f16[n/32], quants i8[n] | covers src.len/32 blocks", launch_kv_quant_q8},
    {"kv_dequant_q8", {256, 1, 1}, 3, 0, "scales f16[n/32], quants i8[n], dst f16[n] | covers dst.len/32 blocks", launch_kv_dequant_q8},

    {"rmsnorm_256", {256, 1, 1}, 3, 0, "x f16[rows x256], w f32[256], y f16 | grid [rows]; y = x * rsqrt(mean(x^2) + 1e-6) * w", launch_rmsnorm<256, 0>},
    {"rmsnorm_256_plus1", {256, 1, 1}, 3, 0, "as rmsnorm_256 with weight 1 + w", launch_rmsnorm<256, 1>},
    {"rmsnorm_512", {256, 1, 1}, 3, 0, "x f16[rows x512], w f32[512], y f16 | grid [rows]", launch_rmsnorm<512, 0>},
    {"rmsnorm_512_plus1", {256, 1, 1}, 3, 0, "as rmsnorm_512 with weight 1 + w", launch_rmsnorm<512, 1>},
    {"rope_sliding_q", {256, 1, 1}, 2, 0, "xs f16[token x32x256] in place, cos_sin f32[token x128 x2] | grid covers rows*128 pairs; pair i = dims (i, i+128)",
     launch_rope<256, 256, 32>},
    {"rope_sliding_k", {256, 1, 1}, 2, 0, "xs f16[token x16x256] in place, cos_sin f32[token x128 x2]", launch_rope<256, 256, 16>},
    {"rope_global_q", {256, 1, 1}, 2, 0, "xs f16[token x32x512] in place, cos_sin f32[token x64 x2] | pair i = dims (i, i+256), i < 64 rotate",
     launch_rope<512, 128, 32>},
    {"rope_global_k", {256, 1, 1}, 2, 0, "xs f16[token x4x512] in place, cos_sin f32[token x64 x2]", launch_rope<512, 128, 4>},

    // ---- head_dim 128, GQA 2, kv heads = groups[0] ------------------------------------------------------
    {"attn_decode_paged_q8kv_d128", {160, 1, 1}, 8, 12,
     "q f16[m_q x H x128], k_quants i8[row x KV x128], k_scales f16[row x KV x4], v_quants, v_scales, page_table u32, "
     "part f32[m_q*H x n_splits x 130], step | push {n_splits u32, scale f32, page u32} | grid [KV, n_splits, m_q<=4 (0/1 = decode)]; "
     "kv_len = step[2]; row = page_table[t/page]*page + t%page; query i sees t <= kv_len - m_q + i",
     launch_decode_paged_q8kv_d128},
    {"attn_verify_paged_q8kv_d128", {160, 1, 1}, 8, 12,
     "as attn_decode_paged_q8kv_d128 with m_q = groups[2] query tokens, causal among themselves (append-then-attend)",
     launch_decode_paged_q8kv_d128},
    {"attn_decode_paged_q8kv_scalar_d128", {128, 1, 1}, 8, 12,
     "same bindings, push and grid as attn_decode_paged_q8kv_d128; one-warp-per-key CUDA-core statement of the same math",
     launch_decode_paged_q8kv_scalar_d128},
    {"attn_decode_sliding_d128", {128, 1, 1}, 5, 8,
     "q f16[H x128], k_ring f16[slot x KV x128], v_ring, part f32[H x n_splits x 130], step | push {n_splits, scale} | "
     "grid [KV, n_splits]; kv_len = step[1]; slots in physical order",
     launch_decode_generic<128, 2, FMT_F16, FMT_F16, SLOT_SLIDING>},
    {"attn_reduce_d128", {128, 1, 1}, 2, 4, "part f32[rows x n_splits x 130], out f16[rows x128] | push {n_splits} | grid [rows]",
     launch_reduce<128, 0>},
    {"attn_reduce_f32_d128", {128, 1, 1}, 2, 4, "part f32[rows x n_splits x 130], out f32[rows x128] | push {n_splits} | grid [rows]",
     launch_reduce<128, 1>},
    {"attn_reduce_partial_d128", {128, 1, 1}, 2, 4,
     "part f32[rows x n_splits x 130], out f32[rows x 130] = merged (acc, m, l), not normalised | push {n_splits} | grid [rows]",
     launch_reduce<128, 2>},
    {"attn_combine_ranks_d128", {128, 1, 1}, 2, 4,
     "gathered f32[n_ranks x rows x 130], out f32[rows x128] | push {n_ranks} | grid [rows]; merged in rank order",
     launch_combine_ranks_d128},
    {"attn_prefill_sliding_f32_d128", {128, 1, 1}, 5, 4,
     "q f16[M x H x128], k f16[token x KV x128], v, out f32[M x H x128], step | push {scale} | grid [KV, M]; window 1024",
     launch_prefill_generic<128, 2, 1024, 0, 0, 1>},
    {"attn_prefill_sliding_ring_f32_d128", {128, 1, 1}, 7, 4,
     "q, k_ring f16[1024 x KV x128], v_ring, k_chunk f16[M x KV x128], v_chunk, out f32, step | push {scale} | grid [KV, M]",
     launch_prefill_generic<128, 2, 1024, 1024, 1, 1>},
    {"attn_verify_sliding_ring_d128", {128, 1, 1}, 7, 4,
     "attn_prefill_sliding_ring_f32_d128 under the name the speculative-verify step uses (M = draft length)",
     launch_prefill_generic<128, 2, 1024, 1024, 1, 1>},
    {"attn_prefill_global_f32_d128", {128, 1, 1}, 5, 4,
     "q f16[M x H x128], k f16[token x KV x128], v, out f32, step | push {scale} | grid [KV, M]; causal [0, q0+i]; scalar",
     launch_prefill_generic<128, 2, 0, 0, 0, 1>},
    {"attn_prefill_paged_q8kv_scalar_d128", {128, 1, 1}, 8, 8,
     "q f16, k_quants, k_scales, v_quants, v_scales, page_table, out f32[M x H x128], step | push {scale f32, page u32} | "
     "grid [KV, M]; causal [0, q0+i]; scalar statement of the paged Q8_0 prefill",
     launch_prefill_paged_q8kv_scalar_d128},
    {"attn_prefill_flash_f16_d128", {128, 1, 1}, 5, 8,
     "q f16[M x H x128], k f16[token x KV x128], v, out f32[M x H x128], step | push {scale f32, window u32 (0 = none)} | "
     "grid [KV, M]; tcgen05 flash attention over linear f16 K/V; q0 = step[3]",
     launch_prefill_flash_f16_d128},
    {"attn_prefill_sliding_ring_flash_d128", {128, 1, 1}, 7, 4,
     "bindings and push of attn_prefill_sliding_ring_f32_d128 | grid [KV, M]; tcgen05 tiles, ring history then chunk",
     launch_prefill_sliding_ring_flash_d128},
    {"attn_prefill_paged_q8kv_flash_d128", {128, 1, 1}, 10, 8,
     "q f16, k_quants, k_scales, v_quants, v_scales, page_table, k_lin f16[rows x KV x128] (scratch), v_lin (scratch), "
     "out f32[M x H x128], step | push {scale f32, page u32} | grid [KV, M]; dequantises the first step[2] tokens into the "
     "linear scratch as f16(scale*q), then runs the tcgen05 flash kernel; causal [0, q0+i]",
     launch_prefill_paged_q8kv_flash_d128},
    {"kv_append_sliding_d128", {256, 1, 1}, 3, 0, "src f16[n x2048], dst f16[1024 x2048], step | slot = (step[0]+token) % 1024",
     launch_kv_append<2048, 1024>},
    {"kv_append_paged_q8_d128", {256, 1, 1}, 5, 8,
     "src f16[n x row_len], scales f16, quants i8, page_table u32, step | push {row_len u32, page u32} | row via page table from step[0]+token",
     launch_kv_append_paged_q8_d128},
    {"attn_reduce_exchange_d128", {64, 1, 1}, 4, 16,
     "part f32[rows x n_splits x 130], xbuf (this rank's exchange buffer: lines u32[2][world][rows][65][4] = {value, epoch, value, epoch}, then u32[rows]; zeroed once), "
     "peers u64[world] (every rank's xbuf, rank order), out f32[rows x128] | push {n_splits u32, world u32, rank u32, wait_us u32 (0 = about a second)} | "
     "grid [rows]; merges the local splits, stores the row into every rank's buffer over NVLink, waits (bounded) for all ranks' rows, merges in "
     "rank order.  After SGB_ERR_TIMEOUT the row's epoch is not advanced: re-zero every rank's xbuf under a host barrier before reuse",
     launch_reduce_exchange_d128},
    {"attn_reduce_exchange_timed_d128", {64, 1, 1}, 5, 16,
     "bindings and push of attn_reduce_exchange_d128, then stamps u64[rows x 5]: GPU global timer (ns) at entry, after the local merge, after the "
     "peer stores and flags, after the wait, at the end",
     launch_reduce_exchange_timed_d128},
    {"attn_norm_rope_d128", {256, 1, 1}, 4, 12,
     "x f16[token x n_heads x128], w f32[128], cos_sin f32[token x rot/2 x2], y f16 | push {n_heads u32, rot_dims u32 (multiple of 16), plus_one u32} | "
     "RMS norm per head, then rotate-half RoPE of the first rot_dims/2 pairs (i, i+64); rounds to f16 after each, like the two-kernel chain",
     launch_norm_rope_d128},
    {"kv_norm_rope_append_paged_q8_d128", {256, 1, 1}, 10, 16,
     "k_raw f16[n x row_len], v_raw, k_w f32[128], cos_sin f32[n x rot/2 x2], k_scales, k_quants, v_scales, v_quants, page_table u32, step | "
     "push {row_len u32, page u32, rot_dims u32, plus_one u32} | K: norm(k_w) + RoPE, V: weightless norm; both Q8_0-quantised into row "
     "page_table[t/page]*page + t%page, t = step[0] + token",
     launch_kv_norm_rope_append_paged_q8_d128},
    {"qkv_norm_rope_append_paged_q8_d128", {256, 1, 1}, 13, 20,
     "q_raw f16[n x n_q x128], q_w f32[128], q_out f16, then the ten bindings of kv_norm_rope_append_paged_q8_d128 | "
     "push {n_q_heads u32, row_len u32, page u32, rot_dims u32, plus_one u32} | the whole pre-attention step in one launch: "
     "q = RoPE(norm(q_raw, q_w)) as f16, and K/V normed, rotated, quantised and appended as by the ten-binding kernel",
     launch_qkv_norm_rope_append_paged_q8_d128},
    {"kv_dequant_paged_q8_d128", {256, 1, 1}, 5, 8,
     "scales f16, quants i8, page_table u32, dst f16[rows x row_len], step | push {row_len, page} | first step[2] tokens, gathered to linear f16; rows up to the next multiple of 64 zeroed",
     launch_kv_dequant_paged_q8_d128},
    // ---- measurement aid -----------------------------------------------------------------------------------------
    {"diag_mma_cycles", {64, 1, 1}, 1, 8,
     "cycles u64[2 x SMs x groups[0]] (per CTA: cycles until n_mma back-to-back tcgen05.mma completed, cycles until they were issued) | "
     "push {shape u32 (0: SS M128xN64xK16, 1: SS M128xN128xK16, 2: TS M128xN128xK16, 3: 8 of shape 1 then 8 of shape 2, repeated), "
     "n_mma u32} | grid [CTAs per SM: 1 or 2, operand data: 0 or 1 = f16 ones, 2 = seeded values in (-1, 1)]; not part of the attention path",
     launch_diag_mma_cycles},
};

}  // namespace

const KernelEntry* registry(int* count)
{
    *count = (int)(sizeof(REGISTRY) / sizeof(REGISTRY[0]));
    return REGISTRY;
}

}  // namespace sgb
