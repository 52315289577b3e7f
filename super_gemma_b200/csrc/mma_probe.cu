// Measurement aid, not part of the attention path: how many SM cycles one tcgen05.mma of the shapes the
// prefill kernels issue takes when nothing but its operands limits it.  Every CTA issues `n_mma`
// instructions back to back from one thread (operands resident in shared / tensor memory, contents
// irrelevant), commits, waits (bounded) and reports clock64() deltas.  Shapes:
//   0  SS  M128 x N64  x K16   (Q K^T with 64-key tiles: 4 KB of A + 2 KB of B from shared memory)
//   1  SS  M128 x N128 x K16   (Q K^T with 128-key tiles: 4 KB + 4 KB)
//   2  TS  M128 x N128 x K16   (P V: A from tensor memory, 4 KB of B from shared memory)
//   3  the 128-key tile's mix: 8 x shape 1, then 8 x shape 2, repeated
// Operand descriptors are built once and stepped by an add, as in the prefill kernels: the figure is the pipe's, not
// the issuing thread's.
// With ctas_per_sm = 2 two CTAs share an SM's tensor pipe, as in the prefill kernels.
#include <string>

#include "sgb_common.cuh"
#include "sgb_kernels.h"

namespace sgb {
namespace {

constexpr uint32_t PROBE_SMEM = 96 * 1024;

template <int SHAPE>
__global__ void __launch_bounds__(64, 2) mma_probe_kernel(uint32_t n_mma, unsigned long long* __restrict__ cycles, uint32_t* status,
                                                          uint32_t random_data)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_base;
    const int tid = threadIdx.x, warp = tid >> 5;
    // operands: f16 1.0 everywhere, or seeded values in (-1, 1): constant operands toggle few wires and draw far less power
    // than real data, so a figure meant to stand for a kernel under the board's power limit needs the second kind.
    // Finite either way: D is overwritten by the first MMA of every group of eight.
    auto operand_word = [&](uint32_t i) -> uint32_t {
        if (!random_data) return 0x3C003C00u;
        uint32_t x = (i + 0x9E3779B9u * (blockIdx.x + 1)) * 2654435761u;
        x ^= x >> 15, x *= 0x2C1B3C6Du, x ^= x >> 12;
        const __half2 h = __floats2half2_rn(((int)(x & 0xffffu) - 32768) * (1.0f / 32768.0f), ((int)(x >> 16) - 32768) * (1.0f / 32768.0f));
        return *reinterpret_cast<const uint32_t*>(&h);
    };
    for (uint32_t i = tid; i < PROBE_SMEM / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_raw)[i] = operand_word(i);
    if (tid == 0) {
        mbar_init(&done_bar, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_base, 256);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base;
    if (warp == 0) {  // the A operand of the TS shapes: 64 columns of packed f16 values
        uint32_t ones[32];
#pragma unroll
        for (int i = 0; i < 32; i++) ones[i] = operand_word(0x40000u + tid * 32 + i);
        tmem_st_32x32b_x32(tmem, ones);
        tmem_st_32x32b_x32(tmem + 32, ones);
        tc_wait_st();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    bool failed = false;
    if (tid == 0) {
        const uint32_t a_base = smem_u32(smem_raw), b_base = a_base + 32768, v_base = a_base + 65536;
        constexpr uint32_t ID_N64 = umma_idesc_f16(128, 64, 0, 0), ID_N128 = umma_idesc_f16(128, 128, 0, 0),
                           ID_PV = umma_idesc_f16(128, 128, 0, 1);
        constexpr uint32_t ID_SS = SHAPE == 0 ? ID_N64 : ID_N128;
        // descriptors built once, stepped by adding to the address field (bytes >> 4), as the prefill kernels do
        const uint64_t da[2] = {umma_desc_sw128(a_base, 16, 1024), umma_desc_sw128(a_base + 16384, 16, 1024)};
        const uint64_t db[2] = {umma_desc_sw128(b_base, 16, 1024), umma_desc_sw128(b_base + 16384, 16, 1024)};
        const uint64_t dv = umma_desc_sw128(v_base, 16384, 1024);
        const long long t0 = clock64();
        for (uint32_t i = 0; i < n_mma; i += 16) {
            if (SHAPE != 2) {
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(tmem, da[0] + 2 * kk, db[0] + 2 * kk, ID_SS, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(tmem, da[1] + 2 * kk, db[1] + 2 * kk, ID_SS, 1u);
            }
            if (SHAPE >= 2) {
#pragma unroll
                for (int kk = 0; kk < 8; kk++) umma_f16_ts(tmem + 128, tmem + kk * 8, dv + 128 * kk, ID_PV, kk ? 1u : 0u);
            }
            if (SHAPE < 2) {
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(tmem, da[0] + 2 * kk, db[0] + 2 * kk, ID_SS, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(tmem, da[1] + 2 * kk, db[1] + 2 * kk, ID_SS, 1u);
            }
            if (SHAPE == 2) {
#pragma unroll
                for (int kk = 0; kk < 8; kk++) umma_f16_ts(tmem + 128, tmem + kk * 8, dv + 128 * kk, ID_PV, kk ? 1u : 0u);
            }
        }
        umma_commit(&done_bar);
        const long long t_issued = clock64();
        mbar_wait(&done_bar, 0, status, 901, failed);
        const long long t1 = clock64();
        cycles[2 * blockIdx.x] = (unsigned long long)(t1 - t0);
        cycles[2 * blockIdx.x + 1] = (unsigned long long)(t_issued - t0);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

struct PushProbe {
    uint32_t shape, n_mma;
};

}  // namespace

// diag_mma_cycles: cycles u64[2 x CTAs] (per CTA: cycles until all MMAs completed, cycles until all were issued).
// push {shape u32, n_mma u32 (multiple of 16)}.  grid [ctas_per_sm (1 or 2), data (0 or 1 = f16 ones, 2 = seeded values
// in (-1, 1))]: SMs x ctas_per_sm CTAs are launched.
int launch_diag_mma_cycles(const LaunchArgs& a)
{
    const PushProbe p = *(const PushProbe*)a.push;
    const uint32_t per_sm = a.groups[0];
    if (p.shape > 3 || p.n_mma == 0 || (p.n_mma & 15) || p.n_mma > (1u << 20) || per_sm < 1 || per_sm > 2)
        return fail_validation(a, "diag_mma_cycles: shape 0..3, n_mma a multiple of 16 up to 2^20, groups[0] = CTAs per SM (1 or 2)");
    const uint32_t ctas = (uint32_t)a.sm_count * per_sm;
    if (int r = need_bytes(a, 0, (size_t)ctas * 16, "cycles")) return r;
    if (a.groups[1] > 2) return fail_validation(a, "diag_mma_cycles: groups[1] = operand data, 0 or 1 (ones) or 2 (seeded values)");
    typedef void (*ProbeKernel)(uint32_t, unsigned long long*, uint32_t*, uint32_t);
    const ProbeKernel kern = p.shape == 0 ? mma_probe_kernel<0> : p.shape == 1 ? mma_probe_kernel<1> : p.shape == 2 ? mma_probe_kernel<2> : mma_probe_kernel<3>;
    if (int r = check_cuda(a, cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PROBE_SMEM),
                           "cudaFuncSetAttribute(mma_probe)"))
        return r;
    kern<<<ctas, 64, PROBE_SMEM, a.stream>>>(p.n_mma, (unsigned long long*)a.b[0].ptr, a.status, a.groups[1] == 2 ? 1u : 0u);
    ++*a.launches;
    return check_cuda(a, cudaGetLastError(), "diag_mma_cycles");
}

}  // namespace sgb
