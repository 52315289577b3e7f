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
#include "attn_merge.cuh"
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

// The wait limit is a launch argument (cycles of the SM clock) so that a host whose ranks may launch far
// apart can raise it; 0 means the library's default of about a second.  After a timeout the row is NaN and
// the row's epoch is NOT advanced: the next launch on this buffer fails fast on the same flag instead of
// overwriting a slot that a slow peer may still read.  The host must then re-zero every rank's exchange
// buffer under a barrier before using it again.
__global__ void __launch_bounds__(HD / 2) reduce_exchange_kernel(const float* __restrict__ part, float* xbuf,
                                                                 const unsigned long long* __restrict__ peers, float* __restrict__ out,
                                                                 uint32_t n_splits, uint32_t world, uint32_t rank, long long wait_cycles,
                                                                 uint32_t* status, unsigned long long* stamps)
{
    __shared__ uint32_t timed_out;
    const size_t row = blockIdx.x, rows = gridDim.x;
    const int t = threadIdx.x, d0 = 2 * t;
    if (t == 0) timed_out = 0;
    unsigned long long t_phase[5];
    if (stamps != nullptr && t == 0) t_phase[0] = globaltimer_ns();

    // ---- 1. the local splits of this row, ascending, running maximum -------------------------------------------
    float acc[2];
    MergeState st = merge_splits_running<HD, 2>(part + row * n_splits * ROWF, ROWF, n_splits, d0, acc);
    if (stamps != nullptr && t == 0) t_phase[1] = globaltimer_ns();

    // ---- 2. hand the merged row to every rank (this one included) ---------------------------------------------
    const size_t flags_off = 2 * (size_t)world * rows * ROWF, epoch_off = flags_off + 2 * (size_t)world * rows;
    uint32_t* my_words = reinterpret_cast<uint32_t*>(xbuf);
    const uint32_t epoch = my_words[epoch_off + row] + 1;  // written only by this row's CTA of the previous launch
    const uint32_t parity = epoch & 1;
    const size_t slot = ((size_t)parity * world + rank) * rows + row;
    for (uint32_t p = 0; p < world; p++) {
        float* dst = reinterpret_cast<float*>(peers[p]) + slot * ROWF;
        *reinterpret_cast<float2*>(dst + d0) = make_float2(acc[0], acc[1]);
        if (t == 0) *reinterpret_cast<float2*>(dst + HD) = make_float2(st.m, st.l);
    }
    __threadfence_system();
    __syncthreads();
    if ((uint32_t)t < world) st_release_sys(reinterpret_cast<uint32_t*>(peers[t]) + flags_off + slot, epoch);
    if (stamps != nullptr && t == 0) t_phase[2] = globaltimer_ns();

    // ---- 3. wait for the same row of every rank, with a limit ----------------------------------------------------
    if ((uint32_t)t < world) {
        const uint32_t* flag = my_words + flags_off + ((size_t)parity * world + t) * rows + row;
        const long long limit = wait_cycles > 0 ? wait_cycles : WAIT_LIMIT_CYCLES;
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != epoch) {
            if (clock64() - t0 > limit) {
                timed_out = 1;
                report_error(status, DEV_ERR_TIMEOUT, 601, (uint32_t)row, (uint32_t)t);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (stamps != nullptr && t == 0) t_phase[3] = globaltimer_ns();

    // ---- 4. merge the ranks in rank order (same arithmetic as the splits; ld.cg: written by other GPUs) ---------
    st = merge_splits_running<HD, 2>(xbuf + ((size_t)parity * world * rows + row) * ROWF, rows * ROWF, world, d0, acc);
    const bool bad = timed_out != 0;
    const float nan = __int_as_float(0x7fc00000);  // a row that gave up is NaN, never stale data
    *reinterpret_cast<float2*>(out + row * HD + d0) = bad ? make_float2(nan, nan) : make_float2(acc[0] / st.l, acc[1] / st.l);
    if (t == 0 && !bad) my_words[epoch_off + row] = epoch;
    if (stamps != nullptr && t == 0) {
        t_phase[4] = globaltimer_ns();
        for (int i = 0; i < 5; i++) stamps[row * 5 + i] = t_phase[i];
    }
}

struct PushExchange {
    uint32_t n_splits, world, rank;
    uint32_t wait_us;  // limit of the wait for the peers in microseconds; 0 = the library's default (about a second)
};

int run_reduce_exchange(const LaunchArgs& a, bool timed)
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
    if (timed)
        if (int r = need_bytes(a, 4, rows * 5 * 8, "stamps")) return r;
    // The wait is counted in SM cycles; 2 cycles per nanosecond bounds the clock from above.
    const long long wait_cycles = (long long)p.wait_us * 2000;
    reduce_exchange_kernel<<<(uint32_t)rows, HD / 2, 0, a.stream>>>((const float*)a.b[0].ptr, (float*)a.b[1].ptr,
                                                                  (const unsigned long long*)a.b[2].ptr, (float*)a.b[3].ptr, p.n_splits,
                                                                  p.world, p.rank, wait_cycles, a.status,
                                                                  timed ? (unsigned long long*)a.b[4].ptr : nullptr);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "attn_reduce_exchange_d128");
}

}  // namespace

// attn_reduce_exchange_d128: part f32[rows x n_splits x 130], xbuf (this rank's exchange buffer), peers u64[world]
// (device pointers to every rank's exchange buffer, own included, in rank order), out f32[rows x 128].
// push {n_splits, world, rank, wait_us}.  grid [rows].
int launch_reduce_exchange_d128(const LaunchArgs& a) { return run_reduce_exchange(a, false); }

// attn_reduce_exchange_timed_d128: the same with a fifth binding, stamps u64[rows x 5]: the GPU's global timer (ns)
// at kernel entry, after the local merge, after the peer stores and flags, after the wait, and at the end.
int launch_reduce_exchange_timed_d128(const LaunchArgs& a) { return run_reduce_exchange(a, true); }

}  // namespace sgb
