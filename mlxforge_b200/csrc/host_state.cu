// Host-side state shared by the launchers: the dependent-launch switch, the per-device SM
// count and the table that says which kernels have been launched.
#include "common.cuh"

unsigned long long g_mf_kernel_launches[MF_K_COUNT] = {};

namespace {
const char* const kNames[MF_K_COUNT] = {
    "stream_rows",      "stream_tmap",      "mid_rows",         "gemm_tc",
    "gemm_tc_swiglu",   "gemm_f32",         "attn_generic", "attn_prefill_mma", "attn_prefill_tc",
    "attn_decode",      "attn_decode_tma",  "attn_decode_tma_merged", "attn_decode_merge",
};
int g_sm_count[MF_MAX_DEVICES] = {};
}  // namespace

int mf_sm_count() {
  const int d = mf_current_device();
  if (d < 0) return 0;
  if (g_sm_count[d] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess) return 0;
    g_sm_count[d] = n;
  }
  return g_sm_count[d];
}

// Number of kernel kinds that are counted, the name of one, and how often it has been launched
// in this process (launches recorded into a CUDA graph count once, replays do not).
MF_API int mf_kernel_kinds() { return MF_K_COUNT; }
MF_API const char* mf_kernel_name(int id) { return id >= 0 && id < MF_K_COUNT ? kNames[id] : ""; }
MF_API long long mf_kernel_launches(int id) {
  return id >= 0 && id < MF_K_COUNT ? (long long)g_mf_kernel_launches[id] : -1;
}
