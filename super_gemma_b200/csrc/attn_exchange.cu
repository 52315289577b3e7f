// Sequence-parallel decode: the split-K combine of one rank fused with the exchange between ranks.
//
// With the KV cache of a long sequence split over GPUs, every rank merges its own splits to one
// (acc[128], m, l) per query row, the ranks exchange those 520-byte rows, and each merges all of them in
// rank order (attn_reduce.wgsl:29-56 is the merge; the reference is single-GPU and has no exchange).  Done
// as reduce + all-gather + combine that is three launches and a collective whose latency, not its 17 KB, sets
// the step time.  attn_reduce_exchange_d128 does it in one launch over peer memory: one CTA of 64 threads per
// row merges the row's local splits (arithmetic of attn_reduce_partial_d128) and hands the result to
// exchange_row (attn_exchange.cuh), which stores it into every rank's buffer over NVLink, waits (bounded) for
// the same row of all ranks and merges them in rank order (arithmetic of attn_combine_ranks_d128).  A row
// depends only on the same row of the other ranks.
#include "attn_exchange.cuh"
#include "sgb_kernels.h"

namespace sgb {

namespace {

constexpr int HD = XCHG_HD;
constexpr int ROWF = XCHG_ROWF;
constexpr int XCHG_MAX_SPLITS = 1024;

// One CTA of 64 threads per row.  The wait limit is a launch argument (cycles of the SM clock) so that a host
// whose ranks may launch far apart can raise it; 0 means the library's default of about a second.
__global__ void __launch_bounds__(HD / 2) reduce_exchange_kernel(const float* __restrict__ part, float* xbuf,
                                                                 const unsigned long long* __restrict__ peers, float* __restrict__ out,
                                                                 uint32_t n_splits, uint32_t world, uint32_t rank, long long wait_cycles,
                                                                 uint32_t* status, unsigned long long* stamps)
{
    __shared__ uint32_t timed_out;
    const size_t row = blockIdx.x, rows = gridDim.x;
    const int t = threadIdx.x;
    if (t == 0) timed_out = 0;
    unsigned long long t_phase[5];
    const bool stamp = stamps != nullptr && t == 0;
    if (stamp) t_phase[0] = globaltimer_ns();
    __syncthreads();
    // the local splits of this row, ascending, running maximum
    float acc[2];
    const MergeState st = merge_splits_running<HD, 2, 3>(part + row * n_splits * ROWF, ROWF, n_splits, 2 * t, acc);
    if (stamp) t_phase[1] = globaltimer_ns();
    exchange_row(acc, st, row, rows, t, 1, &timed_out, xbuf, peers, world, rank, wait_cycles, status, out, stamp ? t_phase + 2 : nullptr);
    if (stamp) {
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
        return fail_validation(a, "attn_reduce_exchange_d128: world in 1..32 and rank < world");
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
