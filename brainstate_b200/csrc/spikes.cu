// Spike-vector preparation: packing to bit words and compaction of the active
// rows into a queue (the list the pre-centric scatter walks).
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

// ---- bool/float -> packed words ---------------------------------------------
// One warp per output word; bit (i % 32) of word (i / 32) is spike i.
template <int FORMAT>
__global__ void __launch_bounds__(256) pack_kernel(const void* __restrict__ spikes, int64_t batch, int64_t n,
                                                   int64_t words, uint32_t* __restrict__ bits) {
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t total = batch * words;
  for (int64_t wd = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; wd < total; wd += nwarps) {
    const int64_t b = wd / words, wi = wd - b * words;
    const int64_t i = wi * 32 + lane;
    const bool on = (i < n) && spike_at<FORMAT>(spikes, b * n + i);
    const uint32_t word = __ballot_sync(0xffffffffu, on);
    if (lane == 0) bits[wd] = word;
  }
}

int launch_pack(const void* spikes, int format, int64_t batch, int64_t n, uint32_t* bits, cudaStream_t st) {
  const int64_t words = (n + 31) / 32;
  const int64_t total = batch * words;
  if (total == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (total + 7) / 8;
  if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
  if (format == BSX_SPK_BOOL8)
    pack_kernel<BSX_SPK_BOOL8><<<(unsigned)blocks, 256, 0, st>>>(spikes, batch, n, words, bits);
  else if (format == BSX_SPK_F32)
    pack_kernel<BSX_SPK_F32><<<(unsigned)blocks, 256, 0, st>>>(spikes, batch, n, words, bits);
  else
    return fail(BSX_ERR_INVALID_ARG, "pack: spike format %d cannot be packed", format);
  BSX_LAUNCH_CHECK("pack_kernel");
  return BSX_OK;
}

// ---- compaction of active rows ------------------------------------------------
// Queue entry = flat position b * n_pre + i of an active spike.  Entries of one
// warp are contiguous; the order between warps follows the atomic counter and is
// not fixed.  The same launch clears the output of the product that follows, so
// no separate memset is needed.
__device__ __forceinline__ uint32_t warp_reserve(uint32_t cnt, int lane, int32_t* counter) {
  uint32_t incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
  uint32_t base = 0;
  if (lane == 31 && total) base = (uint32_t)atomicAdd(counter, (int32_t)total);
  base = __shfl_sync(0xffffffffu, base, 31);
  return base + incl - cnt;
}

__device__ __forceinline__ void zero_span(float* __restrict__ z, int64_t n, int64_t tid, int64_t nthreads) {
  if (!z || n <= 0) return;
  // head to a 16-byte boundary, float4 body, scalar tail
  int64_t head = ((16 - (reinterpret_cast<uintptr_t>(z) & 15)) & 15) >> 2;
  if (head > n) head = n;
  for (int64_t i = tid; i < head; i += nthreads) z[i] = 0.f;
  float4* z4 = reinterpret_cast<float4*>(z + head);
  const int64_t n4 = (n - head) >> 2;
  for (int64_t i = tid; i < n4; i += nthreads) z4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t i = head + (n4 << 2) + tid; i < n; i += nthreads) z[i] = 0.f;
}

// VEC = 4: one 32-bit (BOOL8) or 128-bit (F32) load covers four spikes; the base
// pointer must be aligned accordingly.  VEC = 1: scalar loads.
template <int FORMAT, int VEC>
__global__ void __launch_bounds__(256) compact_kernel(const void* __restrict__ spikes, int64_t total,
                                                      QueueHeader* __restrict__ hdr,
                                                      uint32_t* __restrict__ entries,
                                                      float* __restrict__ zero_ptr, int64_t zero_n) {
  const int lane = threadIdx.x & 31;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  zero_span(zero_ptr, zero_n, tid, nthreads);

  const int64_t groups = (total + VEC - 1) / VEC;
  for (int64_t g0 = tid - lane; g0 < groups; g0 += nthreads) {
    const int64_t g = g0 + lane;
    uint32_t m = 0;  // bit k set: spike g*VEC+k is active
    if (g < groups) {
      const int64_t p = g * VEC;
      if (VEC == 4 && p + 4 <= total) {
        if (FORMAT == BSX_SPK_BOOL8) {
          const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(spikes) + g);
          m = ((v & 0xffu) ? 1u : 0u) | ((v & 0xff00u) ? 2u : 0u) | ((v & 0xff0000u) ? 4u : 0u) |
              ((v & 0xff000000u) ? 8u : 0u);
        } else {
          const float4 v = __ldg(reinterpret_cast<const float4*>(spikes) + g);
          m = (v.x != 0.f ? 1u : 0u) | (v.y != 0.f ? 2u : 0u) | (v.z != 0.f ? 4u : 0u) | (v.w != 0.f ? 8u : 0u);
        }
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k)
          if (p + k < total && spike_at<FORMAT>(spikes, p + k)) m |= 1u << k;
      }
    }
    const uint32_t cnt = __popc(m);
    uint32_t pos = warp_reserve(cnt, lane, &hdr->count);
    while (m) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      entries[pos++] = (uint32_t)(g * VEC + k);
    }
  }
}

// Packed input: one thread per word.
__global__ void __launch_bounds__(256) compact_bits_kernel(const uint32_t* __restrict__ bits, int64_t batch,
                                                           int64_t n_pre, int64_t words,
                                                           QueueHeader* __restrict__ hdr,
                                                           uint32_t* __restrict__ entries,
                                                           float* __restrict__ zero_ptr, int64_t zero_n) {
  const int lane = threadIdx.x & 31;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  zero_span(zero_ptr, zero_n, tid, nthreads);
  const int64_t total = batch * words;
  for (int64_t g0 = tid - lane; g0 < total; g0 += nthreads) {
    const int64_t g = g0 + lane;
    uint32_t m = 0;
    int64_t base_i = 0, b = 0;
    if (g < total) {
      b = g / words;
      const int64_t wi = g - b * words;
      base_i = wi * 32;
      m = __ldg(bits + g);
      const int64_t left = n_pre - base_i;  // valid bits in this word
      if (left < 32) m &= (left <= 0) ? 0u : ((1u << left) - 1u);
    }
    const uint32_t cnt = __popc(m);
    uint32_t pos = warp_reserve(cnt, lane, &hdr->count);
    while (m) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      entries[pos++] = (uint32_t)(b * n_pre + base_i + k);
    }
  }
}

int launch_compact(const void* spikes, int format, int64_t batch, int64_t n_pre, QueueHeader* hdr,
                   uint32_t* entries, float* zero_ptr, int64_t zero_n, cudaStream_t st) {
  const int64_t total = batch * n_pre;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  BSX_CUDA(cudaMemsetAsync(hdr, 0, sizeof(QueueHeader), st));
  // enough threads to cover the larger of the scan and the clear, capped at 8 blocks per SM
  int64_t work = total / 4;
  if (zero_n / 4 > work) work = zero_n / 4;
  int64_t blocks = (work + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
  const unsigned g = (unsigned)blocks;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(spikes);
  if (format == BSX_SPK_BOOL8) {
    if ((addr & 3) == 0)
      compact_kernel<BSX_SPK_BOOL8, 4><<<g, 256, 0, st>>>(spikes, total, hdr, entries, zero_ptr, zero_n);
    else
      compact_kernel<BSX_SPK_BOOL8, 1><<<g, 256, 0, st>>>(spikes, total, hdr, entries, zero_ptr, zero_n);
  } else if (format == BSX_SPK_F32) {
    if ((addr & 15) == 0)
      compact_kernel<BSX_SPK_F32, 4><<<g, 256, 0, st>>>(spikes, total, hdr, entries, zero_ptr, zero_n);
    else
      compact_kernel<BSX_SPK_F32, 1><<<g, 256, 0, st>>>(spikes, total, hdr, entries, zero_ptr, zero_n);
  } else if (format == BSX_SPK_BITS32) {
    compact_bits_kernel<<<g, 256, 0, st>>>(static_cast<const uint32_t*>(spikes), batch, n_pre,
                                           (n_pre + 31) / 32, hdr, entries, zero_ptr, zero_n);
  } else {
    return fail(BSX_ERR_INVALID_ARG, "compact: unknown spike format %d", format);
  }
  BSX_LAUNCH_CHECK("compact_kernel");
  return BSX_OK;
}

__global__ void __launch_bounds__(256) zero_kernel(float* __restrict__ z, int64_t n) {
  zero_span(z, n, (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
}

int launch_zero(float* z, int64_t n, cudaStream_t st) {
  if (n <= 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
  zero_kernel<<<(unsigned)blocks, 256, 0, st>>>(z, n);
  BSX_LAUNCH_CHECK("zero_kernel");
  return BSX_OK;
}

}  // namespace bsx

using namespace bsx;

extern "C" int bsx_pack_spikes(const void* spikes, int spike_format, int64_t batch, int64_t n,
                               uint32_t* bits, bsx_stream_t stream) {
  BSX_TRACE("bsx_pack_spikes");
  if (batch < 0 || n < 0) return fail(BSX_ERR_INVALID_ARG, "bsx_pack_spikes: negative size");
  if (batch == 0 || n == 0) return BSX_OK;
  if (!spikes || !bits) return fail(BSX_ERR_INVALID_ARG, "bsx_pack_spikes: NULL buffer");
  return launch_pack(spikes, spike_format, batch, n, bits, as_stream(stream));
}
