// Shared host/device helpers of the bsx library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "bsx.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "bsx is written for sm_100a (B200) only"
#endif

#include <nvtx3/nvToolsExt.h>

namespace bsx {

// Names the enclosing scope for timeline tools (an NVTX range; a no-op costing a few nanoseconds
// when no tool is attached).  Placed at the top of every compute entry point, so that a trace
// shows which C-ABI call each kernel belongs to — the counterpart of the named scopes the
// reference gets from jax.named_scope around its operators.
struct NvtxScope {
  explicit NvtxScope(const char* name) { nvtxRangePushA(name); }
  ~NvtxScope() { nvtxRangePop(); }
  NvtxScope(const NvtxScope&) = delete;
  NvtxScope& operator=(const NvtxScope&) = delete;
};
#define BSX_TRACE(name) ::bsx::NvtxScope bsx_nvtx_scope_(name)

// ---- host-side error plumbing (thread-local message, integer codes) --------
int fail(int status, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define BSX_CUDA(call)                                          \
  do {                                                          \
    cudaError_t bsx_e_ = (call);                                \
    if (bsx_e_ != cudaSuccess) return ::bsx::cuda_fail(bsx_e_, #call); \
  } while (0)

#define BSX_LAUNCH_CHECK(name)                                  \
  do {                                                          \
    cudaError_t bsx_e_ = cudaGetLastError();                    \
    if (bsx_e_ != cudaSuccess) return ::bsx::cuda_fail(bsx_e_, name); \
  } while (0)

// Validates a connectivity descriptor on the host (pointers, sizes, layout).
int check_conn(const bsx_conn_t* c);
// Number of SMs of the current device (148 on B200); <= 0 on failure.
int sm_count();

inline cudaStream_t as_stream(bsx_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- row addressing shared by the fixed-number and CSR layouts -------------
struct RowMap {
  const int32_t* p32;
  const int64_t* p64;
  int64_t K;
  __device__ __forceinline__ void range(int64_t i, int64_t& s, int64_t& e) const {
    if (p64) {
      s = p64[i];
      e = p64[i + 1];
    } else if (p32) {
      s = p32[i];
      e = p32[i + 1];
    } else {
      s = i * K;
      e = s + K;
    }
  }
};

inline RowMap make_rowmap(const bsx_conn_t* c) {
  RowMap r;
  r.p32 = (c->indptr && !c->indptr_is_64) ? static_cast<const int32_t*>(c->indptr) : nullptr;
  r.p64 = (c->indptr && c->indptr_is_64) ? static_cast<const int64_t*>(c->indptr) : nullptr;
  r.K = c->conn_num;
  return r;
}

// Header of the active-row queue kept at the start of a vecmat workspace.
struct QueueHeader {
  int32_t count;     // number of queued entries
  int32_t pad[3];    // keeps the entries 16-byte aligned
};

#ifdef __CUDACC__
// ---- device helpers ---------------------------------------------------------
__device__ __forceinline__ void red_add(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp adds v (times the weight, if heterogeneous) into out[idx[p]] for every
// entry p of [s, e): scalar head and tail around a body of 128-bit loads.  vec_ok
// says that idx (and w) start on a 16-byte boundary.
template <bool HETERO>
__device__ __forceinline__ void scatter_span(const int32_t* __restrict__ idx, const float* __restrict__ w,
                                             int64_t s, int64_t e, int lane, float v,
                                             float* __restrict__ out, bool vec_ok) {
  if (!vec_ok) {
    for (int64_t p = s + lane; p < e; p += 32)
      red_add(out + __ldg(idx + p), HETERO ? __fmul_rn(v, __ldg(w + p)) : v);
    return;
  }
  // [s, a0) scalar head, [a0, a1) 128-bit body, [a1, e) scalar tail
  int64_t a0 = (s + 3) & ~int64_t(3);
  if (a0 > e) a0 = e;
  int64_t a1 = e & ~int64_t(3);
  if (a1 < a0) a1 = a0;
  const int nh = (int)(a0 - s), nt = (int)(e - a1);
  if (lane < nh + nt) {
    const int64_t p = lane < nh ? s + lane : a1 + (lane - nh);
    red_add(out + __ldg(idx + p), HETERO ? __fmul_rn(v, __ldg(w + p)) : v);
  }
  const int4* __restrict__ idx4 = reinterpret_cast<const int4*>(idx);
  const float4* __restrict__ w4 = reinterpret_cast<const float4*>(w);
  const int64_t q1 = a1 >> 2;
#pragma unroll 2
  for (int64_t q = (a0 >> 2) + lane; q < q1; q += 32) {
    const int4 j = __ldg(idx4 + q);
    if (HETERO) {
      const float4 ww = __ldg(w4 + q);
      red_add(out + j.x, __fmul_rn(v, ww.x));
      red_add(out + j.y, __fmul_rn(v, ww.y));
      red_add(out + j.z, __fmul_rn(v, ww.z));
      red_add(out + j.w, __fmul_rn(v, ww.w));
    } else {
      red_add(out + j.x, v);
      red_add(out + j.y, v);
      red_add(out + j.z, v);
      red_add(out + j.w, v);
    }
  }
}

// 1 where the spike at flat position p is active, for the byte/float formats.
template <int FORMAT>
__device__ __forceinline__ bool spike_at(const void* spikes, int64_t p) {
  if (FORMAT == BSX_SPK_BOOL8) return static_cast<const uint8_t*>(spikes)[p] != 0;
  return static_cast<const float*>(spikes)[p] != 0.0f;
}
#endif

}  // namespace bsx
