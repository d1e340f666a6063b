// Dense event product: y[b, :] = sum over active i of W[i, :]   (W row-major, n_pre x n_post).
//
// One block owns a tile of 1024 output columns of one batch row.  It scans the
// spike row once, keeping the active row numbers in shared memory in ascending
// order, then streams the matching rows of W with 128-bit loads and accumulates
// in registers: no atomics, fixed summation order (ascending i), no workspace.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

constexpr int kDenseThreads = 256;
constexpr int kDenseList = 1024;  // active rows buffered per pass

template <int FORMAT>
__global__ void __launch_bounds__(kDenseThreads)
dense_event_kernel(const void* __restrict__ spikes, const float* __restrict__ W, int64_t n_pre,
                   int64_t n_post, float* __restrict__ out, bool vec_ok) {
  __shared__ int32_t list[kDenseList];
  __shared__ int32_t warp_cnt[kDenseThreads / 32];
  __shared__ int32_t list_n;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t b = blockIdx.y;
  const int64_t col0 = (int64_t)blockIdx.x * (kDenseThreads * 4) + threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int64_t next = 0;  // first spike position not yet scanned
  while (next < n_pre) {
    // ---- fill the list with up to kDenseList active rows, in ascending order
    if (threadIdx.x == 0) list_n = 0;
    __syncthreads();
    while (next < n_pre) {
      const int64_t i = next + threadIdx.x;
      const bool on = (i < n_pre) && spike_at<FORMAT>(spikes, b * n_pre + i);
      const uint32_t m = __ballot_sync(0xffffffffu, on);
      if (lane == 0) warp_cnt[wid] = __popc(m);
      __syncthreads();
      int base = list_n, total = 0;
      for (int k = 0; k < kDenseThreads / 32; ++k) {
        if (k < wid) base += warp_cnt[k];
        total += warp_cnt[k];
      }
      const bool fits = list_n + total <= kDenseList;
      if (fits && on) list[base + __popc(m & ((1u << lane) - 1u))] = (int32_t)i;
      __syncthreads();
      if (!fits) break;  // this chunk of spikes is rescanned in the next pass
      if (threadIdx.x == 0) list_n += total;
      next += kDenseThreads;
      __syncthreads();
      if (list_n == kDenseList) break;
    }
    __syncthreads();
    const int n = list_n;
    // ---- accumulate the listed rows
    if (col0 < n_post) {
      if (vec_ok && col0 + 4 <= n_post) {
#pragma unroll 4
        for (int t = 0; t < n; ++t) {
          const float4 r = __ldg(reinterpret_cast<const float4*>(W + (int64_t)list[t] * n_post + col0));
          acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
        }
      } else {
        for (int t = 0; t < n; ++t) {
          const float* r = W + (int64_t)list[t] * n_post + col0;
          acc.x += __ldg(r);
          if (col0 + 1 < n_post) acc.y += __ldg(r + 1);
          if (col0 + 2 < n_post) acc.z += __ldg(r + 2);
          if (col0 + 3 < n_post) acc.w += __ldg(r + 3);
        }
      }
    }
    __syncthreads();
  }
  if (col0 < n_post) {
    float* o = out + b * n_post + col0;
    o[0] = acc.x;
    if (col0 + 1 < n_post) o[1] = acc.y;
    if (col0 + 2 < n_post) o[2] = acc.z;
    if (col0 + 3 < n_post) o[3] = acc.w;
  }
}

// Weight cotangent of the dense event product: dW[i, :] = sum over the batch rows b with
// spk[b, i] != 0 of ct[b, :], in ascending b (no atomics: deterministic).  One block owns a
// tile of 1024 columns of ONE row i: it lists the batch rows where neuron i fired (a strided
// scan of the spike column, warp ballot) and streams the matching rows of ct with 128-bit
// loads.  Rows that never fired are written as zeros: the kernel is bound by the dW stream.
template <int FORMAT>
__global__ void __launch_bounds__(kDenseThreads)
dense_event_dw_kernel(const void* __restrict__ spikes, const float* __restrict__ ct, int64_t batch,
                      int64_t n_pre, int64_t n_post, float* __restrict__ dw, bool vec_ok) {
  __shared__ int32_t list[kDenseList];
  __shared__ int32_t warp_cnt[kDenseThreads / 32];
  __shared__ int32_t list_n;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t i = blockIdx.y;
  const int64_t col0 = (int64_t)blockIdx.x * (kDenseThreads * 4) + threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int64_t next = 0;
  while (next < batch) {
    if (threadIdx.x == 0) list_n = 0;
    __syncthreads();
    while (next < batch) {
      const int64_t b = next + threadIdx.x;
      const bool on = (b < batch) && spike_at<FORMAT>(spikes, b * n_pre + i);
      const uint32_t m = __ballot_sync(0xffffffffu, on);
      if (lane == 0) warp_cnt[wid] = __popc(m);
      __syncthreads();
      int base = list_n, total = 0;
      for (int k = 0; k < kDenseThreads / 32; ++k) {
        if (k < wid) base += warp_cnt[k];
        total += warp_cnt[k];
      }
      const bool fits = list_n + total <= kDenseList;
      if (fits && on) list[base + __popc(m & ((1u << lane) - 1u))] = (int32_t)b;
      __syncthreads();
      if (!fits) break;
      if (threadIdx.x == 0) list_n += total;
      next += kDenseThreads;
      __syncthreads();
      if (list_n == kDenseList) break;
    }
    __syncthreads();
    const int n = list_n;
    if (col0 < n_post) {
      if (vec_ok && col0 + 4 <= n_post) {
#pragma unroll 4
        for (int t = 0; t < n; ++t) {
          const float4 r = __ldg(reinterpret_cast<const float4*>(ct + (int64_t)list[t] * n_post + col0));
          acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
        }
      } else {
        for (int t = 0; t < n; ++t) {
          const float* r = ct + (int64_t)list[t] * n_post + col0;
          acc.x += __ldg(r);
          if (col0 + 1 < n_post) acc.y += __ldg(r + 1);
          if (col0 + 2 < n_post) acc.z += __ldg(r + 2);
          if (col0 + 3 < n_post) acc.w += __ldg(r + 3);
        }
      }
    }
    __syncthreads();
  }
  if (col0 < n_post) {
    float* o = dw + i * n_post + col0;
    if (vec_ok && col0 + 4 <= n_post) {
      *reinterpret_cast<float4*>(o) = acc;
    } else {
      o[0] = acc.x;
      if (col0 + 1 < n_post) o[1] = acc.y;
      if (col0 + 2 < n_post) o[2] = acc.z;
      if (col0 + 3 < n_post) o[3] = acc.w;
    }
  }
}

// Scalar-weight form of the dense event layer: y[b, :] = r[b] * w with r[b] the number of
// events (count != 0) or the value sum of batch row b.  One block per batch row: reduce, then
// broadcast over the output row.  reduced (may be NULL) also receives r.
template <int FORMAT>
__global__ void __launch_bounds__(kDenseThreads)
dense_scalar_kernel(const void* __restrict__ spikes, int64_t n_pre, int64_t n_post, const float* __restrict__ w,
                    int count_events, float* __restrict__ out, float* __restrict__ reduced) {
  __shared__ float part[kDenseThreads / 32];
  __shared__ float total;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t b = blockIdx.x;
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n_pre; i += kDenseThreads) {
    if (count_events) acc += spike_at<FORMAT>(spikes, b * n_pre + i) ? 1.f : 0.f;
    else acc += (FORMAT == BSX_SPK_F32) ? static_cast<const float*>(spikes)[b * n_pre + i]
                                        : (spike_at<FORMAT>(spikes, b * n_pre + i) ? 1.f : 0.f);
  }
  acc = warp_sum(acc);
  if (lane == 0) part[wid] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < kDenseThreads / 32; ++k) t += part[k];
    total = t;
    if (reduced) reduced[b] = t;
  }
  __syncthreads();
  const float y = __fmul_rn(total, __ldg(w));
  for (int64_t j = threadIdx.x; j < n_post; j += kDenseThreads) out[b * n_post + j] = y;
}

}  // namespace bsx

using namespace bsx;

extern "C" int bsx_dense_event_vecmat(const void* spikes, int spike_format, const float* weight,
                                      int64_t batch, int64_t n_pre, int64_t n_post, float* out,
                                      bsx_stream_t stream) {
  BSX_TRACE("bsx_dense_event_vecmat");
  if (batch < 0 || n_pre < 0 || n_post < 0) return fail(BSX_ERR_INVALID_ARG, "negative size");
  if (batch == 0 || n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  if (n_pre > 0 && (!spikes || !weight)) return fail(BSX_ERR_INVALID_ARG, "NULL input");
  if (batch > 65535) return fail(BSX_ERR_UNSUPPORTED, "batch above 65535");
  if (n_pre > INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "n_pre must fit int32");
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const dim3 grid((unsigned)((n_post + kDenseThreads * 4 - 1) / (kDenseThreads * 4)), (unsigned)batch, 1);
  const bool vec_ok = aligned16(weight) && (n_post % 4 == 0);
  cudaStream_t st = as_stream(stream);
  if (spike_format == BSX_SPK_BOOL8)
    dense_event_kernel<BSX_SPK_BOOL8><<<grid, kDenseThreads, 0, st>>>(spikes, weight, n_pre, n_post, out, vec_ok);
  else if (spike_format == BSX_SPK_F32)
    dense_event_kernel<BSX_SPK_F32><<<grid, kDenseThreads, 0, st>>>(spikes, weight, n_pre, n_post, out, vec_ok);
  else
    return fail(BSX_ERR_INVALID_ARG, "dense event product takes BOOL8 or F32 spikes");
  BSX_LAUNCH_CHECK("dense_event_kernel");
  return BSX_OK;
}

extern "C" int bsx_dense_event_dw(const void* spikes, int spike_format, const float* ct, int64_t batch, int64_t n_pre,
                                  int64_t n_post, float* dw, bsx_stream_t stream) {
  BSX_TRACE("bsx_dense_event_dw");
  if (batch < 0 || n_pre < 0 || n_post < 0) return fail(BSX_ERR_INVALID_ARG, "negative size");
  if (n_pre == 0 || n_post == 0) return BSX_OK;
  if (!dw) return fail(BSX_ERR_INVALID_ARG, "dw is NULL");
  if (batch > 0 && (!spikes || !ct)) return fail(BSX_ERR_INVALID_ARG, "NULL input");
  if (n_pre > 65535) {
    // grid.y carries the row: wider layers take several calls over row ranges of the same arrays
    return fail(BSX_ERR_UNSUPPORTED, "n_pre above 65535: call per row range (the spike column stride stays n_pre)");
  }
  if (batch > INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "batch must fit int32");
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  const dim3 grid((unsigned)((n_post + kDenseThreads * 4 - 1) / (kDenseThreads * 4)), (unsigned)n_pre, 1);
  const bool vec_ok = aligned16(ct) && aligned16(dw) && (n_post % 4 == 0);
  cudaStream_t st = as_stream(stream);
  if (spike_format == BSX_SPK_BOOL8)
    dense_event_dw_kernel<BSX_SPK_BOOL8><<<grid, kDenseThreads, 0, st>>>(spikes, ct, batch, n_pre, n_post, dw, vec_ok);
  else if (spike_format == BSX_SPK_F32)
    dense_event_dw_kernel<BSX_SPK_F32><<<grid, kDenseThreads, 0, st>>>(spikes, ct, batch, n_pre, n_post, dw, vec_ok);
  else
    return fail(BSX_ERR_INVALID_ARG, "dense event cotangent takes BOOL8 or F32 spikes");
  BSX_LAUNCH_CHECK("dense_event_dw_kernel");
  return BSX_OK;
}

extern "C" int bsx_dense_event_scalar(const void* spikes, int spike_format, const float* weight, int float_as_event,
                                      int64_t batch, int64_t n_pre, int64_t n_post, float* out, float* reduced,
                                      bsx_stream_t stream) {
  BSX_TRACE("bsx_dense_event_scalar");
  if (batch < 0 || n_pre < 0 || n_post < 0) return fail(BSX_ERR_INVALID_ARG, "negative size");
  if (batch == 0 || n_post == 0) return BSX_OK;
  if (!out || !weight) return fail(BSX_ERR_INVALID_ARG, "NULL buffer");
  if (n_pre > 0 && !spikes) return fail(BSX_ERR_INVALID_ARG, "NULL input");
  if (batch > INT32_MAX) return fail(BSX_ERR_UNSUPPORTED, "batch must fit int32");
  if (sm_count() <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  cudaStream_t st = as_stream(stream);
  const int count = float_as_event ? 1 : 0;
  if (spike_format == BSX_SPK_BOOL8)
    dense_scalar_kernel<BSX_SPK_BOOL8><<<(unsigned)batch, kDenseThreads, 0, st>>>(spikes, n_pre, n_post, weight, count, out, reduced);
  else if (spike_format == BSX_SPK_F32)
    dense_scalar_kernel<BSX_SPK_F32><<<(unsigned)batch, kDenseThreads, 0, st>>>(spikes, n_pre, n_post, weight, count, out, reduced);
  else
    return fail(BSX_ERR_INVALID_ARG, "dense event product takes BOOL8 or F32 spikes");
  BSX_LAUNCH_CHECK("dense_scalar_kernel");
  return BSX_OK;
}
