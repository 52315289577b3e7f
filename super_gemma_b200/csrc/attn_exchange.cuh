// The exchange of one merged row between the ranks of a sequence-parallel decode, as a device function.
// A GROUP of 64 threads (two whole warps) holds the row's locally merged (acc, m, l), two dims per thread, and
//   1. stores it into slot [parity][rank][row] of EVERY rank's exchange buffer with plain peer stores over
//      NVLink.  Every 16-byte store carries two values and, next to each, the row's epoch:
//      {value, epoch, value, epoch}.  The receiver needs no separate flag and the sender no fence: a line is
//      complete when both of its epochs match, and an aligned 16-byte store does not tear within an 8-byte
//      half.  (The form with data, a system-scope fence and a flag store spent 7 of its 15 us in the fence.)
//   2. polls (bounded; DEV_ERR_TIMEOUT after the limit) its own buffer until the lines of all ranks for this
//      row carry the epoch;
//   3. merges the ranks' rows in rank order (merge_batch, the arithmetic of every other combine) and writes
//      out = acc / l.
// Exchange buffer of one rank, in 4-byte words: lines u32[2][world][rows][65][4], then epoch u32[rows];
// zeroed once before first use, after all ranks have allocated theirs (epochs start at 1, so a zeroed line
// never matches).  Slots alternate with the parity of the per-row epoch: a rank can be at most one step
// ahead of a peer that still reads the other parity, because its next step needs that peer's row of the
// current one.  After a timeout the row is NaN and the row's epoch is NOT advanced: the next launch on this
// buffer fails fast on the same lines instead of overwriting a slot that a slow peer may still read; the
// host must then re-zero every rank's buffer under a barrier before using it again.  No multimem, no TMA.
#pragma once

#include "attn_merge.cuh"
#include "sgb_common.cuh"

namespace sgb {

constexpr int XCHG_HD = 128;
constexpr int XCHG_ROWF = XCHG_HD + 2;
constexpr int XCHG_LINES = XCHG_ROWF / 2;  // 16-byte lines per row: 64 of acc, 1 of (m, l)
constexpr int XCHG_MAX_RANKS = 32;         // one lane per rank in the merge

__host__ __device__ inline size_t xchg_words(size_t world, size_t rows) { return 2 * world * rows * XCHG_LINES * 4 + rows; }

__device__ __forceinline__ void st_line(uint4* p, uint32_t a, uint32_t b, uint32_t epoch)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(epoch), "r"(b), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// t = 0..63 is the thread's index in its group, bar_id a named barrier no other group of the CTA uses,
// timed_out a shared-memory word of the group that is zero on entry.  t_phase (thread 0 of the group, may be
// nullptr) receives the global timer after step 1 and after step 2.
__device__ __forceinline__ void exchange_row(const float (&acc_in)[2], MergeState st_in, size_t row, size_t rows, int t, uint32_t bar_id,
                                             uint32_t* timed_out, float* xbuf, const unsigned long long* __restrict__ peers,
                                             uint32_t world, uint32_t rank, long long wait_cycles, uint32_t* status,
                                             float* __restrict__ out, unsigned long long* t_phase)
{
    constexpr int HD = XCHG_HD;
    const uint32_t lane = (uint32_t)t & 31u;
    uint32_t* my_words = reinterpret_cast<uint32_t*>(xbuf);
    const size_t epoch_off = 2 * (size_t)world * rows * XCHG_LINES * 4;
    const uint32_t epoch = __ldcg(my_words + epoch_off + row) + 1;  // written only by this row's group of the previous launch
    const uint32_t parity = epoch & 1;
    // line index of (parity, source rank, row, line)
    auto line_at = [&](uint32_t src, uint32_t line) { return (((size_t)parity * world + src) * rows + row) * XCHG_LINES + line; };

    // ---- 1. my row to every rank (this one included) ----
    for (uint32_t p = 0; p < world; p++) {
        uint4* dst = reinterpret_cast<uint4*>(peers[p]) + line_at(rank, 0);
        st_line(dst + t, __float_as_uint(acc_in[0]), __float_as_uint(acc_in[1]), epoch);
        if (t == 0) st_line(dst + XCHG_LINES - 1, __float_as_uint(st_in.m), __float_as_uint(st_in.l), epoch);
    }
    if (t_phase != nullptr && t == 0) t_phase[0] = globaltimer_ns();

    // ---- 2. every rank's row out of my own buffer: lane u of each warp takes (m, l) of rank u, every thread its two
    //         dims of every rank; a line is there once both of its epochs match ----
    const uint4* mine = reinterpret_cast<const uint4*>(xbuf);
    const long long limit = wait_cycles > 0 ? wait_cycles : WAIT_LIMIT_CYCLES;
    const long long t0 = clock64();
    bool gave_up = false;
    float v[32][2];
    float2 ml = make_float2(NEG_SENTINEL, 0.0f);
#pragma unroll 1
    for (uint32_t s = 0; s < world; s++) {
        const uint4* src = mine + line_at(s, 0);
        uint4 a = ld_line(src + t);
        uint4 b = make_uint4(0u, epoch, 0u, epoch);
        if (lane == s) b = ld_line(src + XCHG_LINES - 1);
        while (!gave_up && (a.y != epoch || a.w != epoch || b.y != epoch || b.w != epoch)) {
            if (clock64() - t0 > limit) {
                gave_up = true;
                *timed_out = 1;
                report_error(status, DEV_ERR_TIMEOUT, 601, (uint32_t)row, s);
                break;
            }
            __nanosleep(40);
            if (a.y != epoch || a.w != epoch) a = ld_line(src + t);
            if (lane == s && (b.y != epoch || b.w != epoch)) b = ld_line(src + XCHG_LINES - 1);
        }
        // registers are indexed statically: rank s goes to slot s of the batch through a switch-free copy below
#pragma unroll
        for (int u = 0; u < 32; u++) {
            if ((uint32_t)u == s) {
                v[u][0] = __uint_as_float(a.x);
                v[u][1] = __uint_as_float(a.z);
            }
        }
        if (lane == s) ml = make_float2(__uint_as_float(b.x), __uint_as_float(b.z));
    }
    named_barrier_sync(bar_id, 64);  // a timeout seen by one thread of the group is seen by all below
    if (t_phase != nullptr && t == 0) t_phase[1] = globaltimer_ns();

    // ---- 3. merge in rank order ----
    float m = NEG_SENTINEL, l = 0.0f, acc[2] = {0.0f, 0.0f};
    merge_batch<2>(v, ml, world, m, l, acc);
    const bool bad = *reinterpret_cast<volatile uint32_t*>(timed_out) != 0;
    const float nan = __int_as_float(0x7fc00000);  // a row that gave up is NaN, never stale data
    *reinterpret_cast<float2*>(out + row * HD + 2 * t) = bad ? make_float2(nan, nan) : make_float2(acc[0] / l, acc[1] / l);
    if (t == 0 && !bad) my_words[epoch_off + row] = epoch;
}

}  // namespace sgb
