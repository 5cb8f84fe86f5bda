// Shared helpers for the sm_100a kernels of mlxforge_b200.
//
// Conventions used by every entry point:
//  * entry points are extern "C", take raw device pointers and the CUDA stream
//    to launch on, allocate nothing, and return a cudaError_t code (0 = ok) or
//    one of the MF_ERR_* codes below for an argument the kernel refuses;
//  * `dtype` arguments are 0 for IEEE float32 and 1 for bfloat16;
//  * matrices are row-major; weights are [out, in] as in the checkpoint.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MF_F32 0
#define MF_BF16 1

#define MF_ERR_BAD_ARG 10001      // a size the kernel does not take
#define MF_ERR_BAD_DTYPE 10002

#define MF_API extern "C" __attribute__((visibility("default")))

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `red` is 32 floats of shared
// memory.  Every thread gets the result.  The order of additions depends only on
// the block size, never on what else runs.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// Paged cache addressing.  One pool per cache lane (a layer's keys or values):
// [page][kv_head][slot][head_dim].  `block_table` holds, per sequence of the
// step, the page of every logical block; entries of blocks that were given back
// (outside a window) are negative and are never addressed.
struct PagedView {
  const int* block_table;   // [n_seqs, bt_stride]
  int bt_stride;
  int page_size;
  int n_kv_heads;
  int head_dim;
};
__device__ __forceinline__ long long paged_offset(const PagedView& pv, int seq, int pos, int kv_head) {
  const int blk = pos / pv.page_size, slot = pos - blk * pv.page_size;
  const long long page = pv.block_table[(long long)seq * pv.bt_stride + blk];
  return ((page * pv.n_kv_heads + kv_head) * pv.page_size + slot) * (long long)pv.head_dim;
}

// Offset of the first of 16 consecutive positions [pos16, pos16 + 16), pos16 a multiple
// of 16: they share a page because the page size is a multiple of 16.  Rows of the
// granule are head_dim apart.  Kernels look this up once per granule and not once per
// row, so that no address waits on a load of the block table inside a copy loop.
__device__ __forceinline__ long long granule_offset(const PagedView& pv, int seq, int pos16, int kv_head) {
  return paged_offset(pv, seq, pos16, kv_head);
}

// ---------------------------------------------------------------------------- dependent launch
// Kernels of the decode step are launched so that the next kernel may start while this
// one is still running (programmatic dependent launch).  A kernel lets its own dependents go
// (pdl_launch), does what needs no input from its predecessor (fetching weights, which never
// change, and keys that earlier steps wrote) and waits for the predecessor to finish (pdl_wait)
// before it reads an activation or writes anything, so the result is that of running the
// kernels one after the other.  The streamed products and the small kernels between them let
// their dependents go FIRST: the blocks of the kernels that follow then take an SM's room the
// moment a block of the running kernel leaves it and fill their rings while the rest of that
// kernel and the small kernel after it finish (1.125 -> 1.095 ms for a decode step of batch 8).
// A dependent starts only when every block of its predecessor has let it go, that is when all
// of them are resident or done, so no kernel can wait for one that has no room to start.  The
// first kernel of a step (the embedding) waits before it lets go: nothing of a step starts
// before the step's inputs are in place.  Under a normal launch both are no-ops.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

extern int g_mf_pdl;      // 1: launch with the dependent-launch attribute (set by mf_set_pdl)

// ---------------------------------------------------------------------------- per-device set-up
// cudaFuncSetAttribute and the SM count belong to a device, not to the process: a launcher keeps
// one flag per device ordinal (a function-local `static DeviceOnce`) and asks which device is
// current.  Ordinals beyond the table are refused by the launcher (MF_ERR_BAD_ARG).
#define MF_MAX_DEVICES 64
struct DeviceOnce {
  bool done[MF_MAX_DEVICES] = {};
};
inline int mf_current_device() {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MF_MAX_DEVICES) return -1;
  return d;
}
// SMs of the current device (looked up once per device); 0 if it cannot be had
int mf_sm_count();

// ---------------------------------------------------------------------------- which kernels ran
// Every launcher counts the kernel it launches (also while a stream is capturing), so that a test
// of a whole model can say which kernels its steps went through: mf_kernel_launches(id).
enum MfKernel {
  MF_K_STREAM_ROWS = 0,       // few-row product, row-segment copies
  MF_K_STREAM_TMAP,           // few-row product, one tensor copy per stage
  MF_K_MID_ROWS,              // product of 17..128 rows (tcgen05, weights on the M side)
  MF_K_GEMM_TC,               // many-row product, tcgen05
  MF_K_GEMM_TC_SWIGLU,        // the same with the gated epilogue
  MF_K_GEMM_F32,
  MF_K_ATTN_GENERIC,
  MF_K_ATTN_PREFILL_MMA,
  MF_K_ATTN_PREFILL_TC,
  MF_K_ATTN_DECODE,           // split-key decode attention without tensor copies
  MF_K_ATTN_DECODE_TMA,       // with tensor copies, a merge kernel after it
  MF_K_ATTN_DECODE_TMA_MERGED,  // with tensor copies, merging its splits itself
  MF_K_ATTN_DECODE_MERGE,
  MF_K_COUNT
};
extern unsigned long long g_mf_kernel_launches[MF_K_COUNT];
inline void mf_count(MfKernel k) { g_mf_kernel_launches[k]++; }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_mf_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
