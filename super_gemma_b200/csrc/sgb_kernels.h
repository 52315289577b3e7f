// Internal: what a registry entry is and the launchers each .cu file provides.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace sgb {

struct BufView {
    void* ptr;
    size_t bytes;
};

struct LaunchArgs {
    cudaStream_t stream;
    const BufView* b;    // bindings, dense, index == position
    const void* push;    // push-constant bytes (already size-checked against the entry)
    uint32_t groups[3];  // the reference's workgroup grid for this kernel
    uint32_t* status;    // device status word (4 x u32) for DEV_ERR_* reports
    int sm_count;
    int device;
    std::string* err;    // filled on validation failure
    uint64_t* launches;  // incremented once per kernel launched
};

typedef int (*LaunchFn)(const LaunchArgs&);

struct KernelEntry {
    const char* name;
    uint32_t workgroup[3];
    uint32_t bindings;
    uint32_t push_bytes;
    const char* signature;
    LaunchFn fn;
};

// Host-side error helpers shared by the launchers (defined in sgb_runtime.cu).
int set_last_error(int code, const std::string& msg);  // records the text sgb_last_error() returns; returns code
int fail_validation(const LaunchArgs& a, const std::string& msg);
int check_cuda(const LaunchArgs& a, cudaError_t e, const char* what);
int need_bytes(const LaunchArgs& a, int binding, size_t bytes, const char* what);

// Tensor-map encoder resolved at run time through the CUDA runtime (no link-time libcuda).
// dims/strides innermost first; strides[i] is the byte stride of dimension i+1.
int encode_tensor_map(const LaunchArgs& a, void* out_map /*CUtensorMap*/, int elem_kind /*0 = u8, 1 = f16*/, int rank,
                      void* base, const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      int swizzle /*0 none, 3 = 128B*/);

// Launch `kern` so that it may overlap the tail of its predecessor in the stream (programmatic dependent
// launch); the kernel calls pdl_wait() before reading.  SGB_PDL=0 in the environment turns the attribute off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The registry (sgb_registry.cu).
const KernelEntry* registry(int* count);

// ---- launchers ------------------------------------------------------------------------------------
// kv_codec.cu
int launch_kv_quant_q8(const LaunchArgs&);
int launch_kv_dequant_q8(const LaunchArgs&);
template <int ROW_LEN, int RING> int launch_kv_append(const LaunchArgs&);
template <int ROW_LEN> int launch_kv_append_global_q8(const LaunchArgs&);
int launch_kv_append_paged_q8_d128(const LaunchArgs&);
int launch_kv_dequant_paged_q8_d128(const LaunchArgs&);

// pre_attn.cu
template <int ROW_LEN, int PLUS_ONE> int launch_rmsnorm(const LaunchArgs&);
template <int HEAD_DIM, int ROT_DIMS, int N_HEADS> int launch_rope(const LaunchArgs&);
int launch_norm_rope_d128(const LaunchArgs&);
int launch_kv_norm_rope_append_paged_q8_d128(const LaunchArgs&);
int launch_qkv_norm_rope_append_paged_q8_d128(const LaunchArgs&);

// attn_generic.cu
template <int HD, int G, int KFMT, int VFMT, int STEP_SLOT> int launch_decode_generic(const LaunchArgs&);
int launch_decode_paged_q8kv_scalar_d128(const LaunchArgs&);
template <int HD, int OUT_MODE> int launch_reduce(const LaunchArgs&);
int launch_combine_ranks_d128(const LaunchArgs&);
template <int HD, int G, int WINDOW, int RING, int TWO_RANGE, int OUT_F32> int launch_prefill_generic(const LaunchArgs&);
int launch_prefill_paged_q8kv_scalar_d128(const LaunchArgs&);
template <int VARIANT> int launch_prefill_global_flash_ref(const LaunchArgs&);

// attn_exchange.cu
int launch_reduce_exchange_d128(const LaunchArgs&);
int launch_reduce_exchange_timed_d128(const LaunchArgs&);

// attn_decode_paged.cu
int launch_decode_paged_q8kv_d128(const LaunchArgs&);

// attn_prefill_flash.cu
int launch_prefill_flash_f16_d128(const LaunchArgs&);
int launch_prefill_sliding_ring_flash_d128(const LaunchArgs&);
int launch_prefill_paged_q8kv_flash_d128(const LaunchArgs&);

// mma_probe.cu
int launch_diag_mma_cycles(const LaunchArgs&);

}  // namespace sgb
