// Sequence-parallel decode: the split-K combine of one rank fused with the exchange between ranks.
//
// With the KV cache of a long sequence split over GPUs, every rank merges its own splits to one
// (acc[128], m, l) per query row, the ranks exchange those 520-byte rows, and each merges all of them in
// rank order (attn_reduce.wgsl:29-56 is the merge; the reference is single-GPU and has no exchange).  Done
// as reduce + all-gather + combine that is three launches and a collective whose latency, not its 17 KB, sets
// the step time.  attn_reduce_exchange_d128 does it in one launch over peer memory:
//   1. merge the local splits of row r                                   (arithmetic of attn_reduce_partial_d128)
//   2. store the merged row into slot [parity][my rank][r] of EVERY rank's exchange buffer with plain peer
//      stores over NVLink, fence, then release-store the step's epoch into that slot's flag
//   3. acquire-poll the local flags of all ranks for row r (bounded: about a second, then DEV_ERR_TIMEOUT)
//   4. merge the ranks' rows in rank order and write out                 (arithmetic of attn_combine_ranks_d128)
// One CTA per row, so a row depends only on the same row of the other ranks.  Slots alternate with the parity
// of a per-row epoch kept in the buffer: a rank can be at most one step ahead of a peer that still reads the
// other parity, because its next step needs that peer's row of the current one.  The buffer must be zeroed
// once, before the first use and after all ranks have allocated it.  No multimem, no TMA: plain ld/st.
#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int HD = 128;
constexpr int ROWF = HD + 2;
constexpr int XCHG_MAX_SPLITS = 1024;
constexpr int XCHG_MAX_RANKS = 64;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Exchange buffer of one rank, in 4-byte words: data f32[2][world][rows][130], flags u32[2][world][rows],
// epoch u32[rows].
__host__ __device__ inline size_t xchg_words(size_t world, size_t rows) { return 2 * world * rows * ROWF + 2 * world * rows + rows; }

__global__ void __launch_bounds__(128) reduce_exchange_kernel(const float* __restrict__ part, float* xbuf,
                                                              const unsigned long long* __restrict__ peers, float* __restrict__ out,
                                                              uint32_t n_splits, uint32_t world, uint32_t rank, uint32_t* status)
{
    __shared__ float w_s[XCHG_MAX_SPLITS];
    __shared__ float wl_s[XCHG_MAX_SPLITS];
    __shared__ float red[4];
    __shared__ uint32_t timed_out;
    const size_t row = blockIdx.x, rows = gridDim.x;
    const int t = threadIdx.x;
    if (t == 0) timed_out = 0;

    // ---- 1. the local splits of this row: M = max m_s, acc = sum exp(m_s - M) acc_s, l likewise, ascending s ----
    const float* base = part + row * n_splits * ROWF;
    float mx = NEG_SENTINEL;
    for (uint32_t s = t; s < n_splits; s += 128) {
        const float ms = base[s * ROWF + HD];
        w_s[s] = ms;
        wl_s[s] = base[s * ROWF + HD + 1];
        mx = fmaxf(mx, ms);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((t & 31) == 0) red[t >> 5] = mx;
    __syncthreads();
    const float m_loc = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    for (uint32_t s = t; s < n_splits; s += 128) {
        const float w = __expf(w_s[s] - m_loc);  // empty split: exp(-3e38 - m) = 0
        w_s[s] = w;
        wl_s[s] *= w;
    }
    __syncthreads();
    float acc = 0.0f, l = 0.0f;
    for (uint32_t s = 0; s < n_splits; s++) {
        acc = fmaf(w_s[s], base[s * ROWF + t], acc);
        l += wl_s[s];
    }

    // ---- 2. hand the merged row to every rank (this one included) ---------------------------------------------
    const size_t flags_off = 2 * (size_t)world * rows * ROWF, epoch_off = flags_off + 2 * (size_t)world * rows;
    uint32_t* my_words = reinterpret_cast<uint32_t*>(xbuf);
    const uint32_t epoch = my_words[epoch_off + row] + 1;  // written only by this row's CTA of the previous launch
    const uint32_t parity = epoch & 1;
    const size_t slot = ((size_t)parity * world + rank) * rows + row;
    for (uint32_t p = 0; p < world; p++) {
        float* dst = reinterpret_cast<float*>(peers[p]) + slot * ROWF;
        dst[t] = acc;
        if (t == 0) {
            dst[HD] = m_loc;
            dst[HD + 1] = l;
        }
    }
    __threadfence_system();
    __syncthreads();
    if ((uint32_t)t < world) st_release_sys(reinterpret_cast<uint32_t*>(peers[t]) + flags_off + slot, epoch);

    // ---- 3. wait for the same row of every rank, with a limit ----------------------------------------------------
    if ((uint32_t)t < world) {
        const uint32_t* flag = my_words + flags_off + ((size_t)parity * world + t) * rows + row;
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != epoch) {
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                timed_out = 1;
                report_error(status, DEV_ERR_TIMEOUT, 601, (uint32_t)row, (uint32_t)t);
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();

    // ---- 4. merge the ranks in rank order (same arithmetic as the splits) ---------------------------------------
    const float* gathered = xbuf + ((size_t)parity * world * rows + row) * ROWF;  // + src * rows * ROWF
    const size_t r_stride = rows * ROWF;
    mx = NEG_SENTINEL;
    if ((uint32_t)t < world) {
        w_s[t] = __ldcg(gathered + t * r_stride + HD);  // written by another GPU: never from this SM's L1
        wl_s[t] = __ldcg(gathered + t * r_stride + HD + 1);
        mx = w_s[t];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __syncthreads();  // red[] was read above by all threads
    if ((t & 31) == 0) red[t >> 5] = mx;
    __syncthreads();
    const float m_all = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    if ((uint32_t)t < world) {
        const float w = __expf(w_s[t] - m_all);
        w_s[t] = w;
        wl_s[t] *= w;
    }
    __syncthreads();
    acc = 0.0f;
    l = 0.0f;
    for (uint32_t s = 0; s < world; s++) {
        acc = fmaf(w_s[s], __ldcg(gathered + s * r_stride + t), acc);
        l += wl_s[s];
    }
    out[row * HD + t] = timed_out ? __int_as_float(0x7fc00000) : acc / l;  // a row that gave up is NaN, never stale data
    if (t == 0) my_words[epoch_off + row] = epoch;
}

struct PushExchange {
    uint32_t n_splits, world, rank;
};

}  // namespace

// attn_reduce_exchange_d128: part f32[rows x n_splits x 130], xbuf (this rank's exchange buffer), peers u64[world]
// (device pointers to every rank's exchange buffer, own included, in rank order), out f32[rows x 128].
// push {n_splits, world, rank}.  grid [rows].
int launch_reduce_exchange_d128(const LaunchArgs& a)
{
    const PushExchange p = *(const PushExchange*)a.push;
    const size_t rows = a.groups[0];
    if (rows == 0 || p.n_splits == 0 || p.n_splits > (uint32_t)XCHG_MAX_SPLITS)
        return fail_validation(a, "attn_reduce_exchange_d128: groups[0] (rows) must be > 0 and n_splits in 1..1024");
    if (p.world == 0 || p.world > (uint32_t)XCHG_MAX_RANKS || p.rank >= p.world)
        return fail_validation(a, "attn_reduce_exchange_d128: world in 1..64 and rank < world");
    if (int r = need_bytes(a, 0, rows * p.n_splits * ROWF * 4, "part")) return r;
    if (int r = need_bytes(a, 1, xchg_words(p.world, rows) * 4, "exchange buffer")) return r;
    if (int r = need_bytes(a, 2, (size_t)p.world * 8, "peers")) return r;
    if (int r = need_bytes(a, 3, rows * HD * 4, "out")) return r;
    reduce_exchange_kernel<<<(uint32_t)rows, 128, 0, a.stream>>>((const float*)a.b[0].ptr, (float*)a.b[1].ptr,
                                                               (const unsigned long long*)a.b[2].ptr, (float*)a.b[3].ptr, p.n_splits,
                                                               p.world, p.rank, a.status);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_reduce_exchange_d128");
}

}  // namespace sgb
