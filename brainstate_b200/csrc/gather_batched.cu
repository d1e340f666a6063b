// Batched event matvec: y[b, i] = sum_k w[i,k] * [s[b, idx[i,k]] != 0] for up to 16
// spike vectors per pass over the indices.
//
// One pass reads every index once and tests it against the spikes of 16 vectors
// at a time: the spikes are transposed into one 16-bit word per column (bit b =
// vector b), staged whole into shared memory by a bulk-async (TMA) copy.  A warp
// owns a row: it compacts the entries whose word is nonzero into a short list in
// shared memory (__ballot_sync / __popc), fetches their weights together, then
// walks the list with one lane per (half of the list, vector).  No atomics, fixed
// summation order: deterministic.  HBM traffic per pass: 4 B per stored synapse
// + 4 B per (hit, heterogeneous weight), shared by 16 vectors.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

constexpr int kB16Threads = 1024;
constexpr int kB16 = 16;
constexpr int kB16List = 256;  // hits buffered per warp before they are consumed (even)

// ---- spikes (batch, n) -> one 16-bit word per column and group of 16 vectors -------
template <int FORMAT>
__global__ void __launch_bounds__(256)
pack16_kernel(const void* __restrict__ spikes, int64_t batch, int64_t n, int64_t n_pad,
              uint16_t* __restrict__ masks, int32_t* __restrict__ nonzero_words) {
  const int64_t groups = (batch + kB16 - 1) / kB16;
  const int64_t total = groups * n_pad;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t words = (n + 31) >> 5;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t g = t / n_pad, j = t - g * n_pad;
    uint32_t m = 0;
    if (j < n) {
#pragma unroll
      for (int b = 0; b < kB16; ++b) {
        const int64_t row = g * kB16 + b;
        if (row < batch) {
          bool on;
          if (FORMAT == BSX_SPK_BITS32)
            on = (static_cast<const uint32_t*>(spikes)[row * words + (j >> 5)] >> (j & 31)) & 1u;
          else
            on = spike_at<FORMAT>(spikes, row * n + j);
          m |= (uint32_t)on << b;
        }
      }
    }
    masks[t] = (uint16_t)m;
    // per group: how many columns carry a spike of any of the 16 vectors; the gather
    // reads this to estimate the fraction of synapses that will hit
    const uint32_t any = __ballot_sync(__activemask(), m != 0);
    if (m != 0 && (threadIdx.x & 31) == (__ffs(any) - 1)) atomicAdd(nonzero_words + g, __popc(any));
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Stages `bytes` (a multiple of 16, source 16-byte aligned) into shared memory with
// bulk-async copies on an mbarrier; bounded wait, plain-load fallback.
__device__ __forceinline__ void stage_bytes(void* __restrict__ smem, const void* __restrict__ gmem, uint32_t bytes,
                                            bool use_tma, uint64_t* bar) {
  bool done = false;
  if (use_tma) {
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(1) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                   : "memory");
      const uint32_t piece = 32768;
      for (uint32_t off = 0; off < bytes; off += piece) {
        const uint32_t sz = bytes - off < piece ? bytes - off : piece;
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_addr(static_cast<char*>(smem) + off)),
            "l"(static_cast<const char*>(gmem) + off), "r"(sz), "r"(smem_addr(bar))
            : "memory");
      }
    }
    bool ok = false;
    for (int spin = 0; spin < (1 << 22) && !ok; ++spin) {
      uint32_t r;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(r)
          : "r"(smem_addr(bar)), "r"(0)
          : "memory");
      ok = r != 0;
    }
    done = __syncthreads_and(ok);
  }
  if (!done) {
    const uint4* src = static_cast<const uint4*>(gmem);
    uint4* dst = static_cast<uint4*>(smem);
    for (uint32_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) dst[i] = __ldg(src + i);
    __syncthreads();
  }
}

// Body of the kernel for one way of reading the weights (EAGER: streamed with the
// indices; otherwise fetched per hit).  All loop arithmetic inside a row is 32-bit and
// relative to the row start.
template <bool HETERO, bool EAGER>
__device__ __forceinline__ void b16_rows(const RowMap& rm, const int32_t* __restrict__ idx,
                                         const float* __restrict__ w, const uint16_t* __restrict__ smask,
                                         uint2* __restrict__ list, int64_t n_rows, float* __restrict__ out,
                                         int nb, bool vec_ok, float w0) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  const int b = lane & 15, half = lane >> 4;
  const uint4* __restrict__ pairs = reinterpret_cast<const uint4*>(list);
  const int64_t wstep = (int64_t)gridDim.x * (kB16Threads >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (kB16Threads >> 5) + wid; row < n_rows; row += wstep) {
    int64_t s, e;
    rm.range(row, s, e);
    const int len = (int)(e - s);
    const int32_t* __restrict__ ri = idx + s;
    const float* __restrict__ rw = w + s;
    int head = len, nvec = 0;                        // unaligned arrays: everything is "head"
    if (vec_ok) {
      head = (int)((4 - (s & 3)) & 3);
      if (head > len) head = len;
      nvec = (len - head) >> 2;
    }
    const int tail0 = head + (nvec << 2);            // first entry after the 128-bit body
    const int4* __restrict__ r4 = reinterpret_cast<const int4*>(ri + head);
    const float4* __restrict__ rw4 = reinterpret_cast<const float4*>(rw + head);
    int n_list = 0;
    float acc = 0.f;

#define BSX_B16_PUSH(VALID, J, PAYLOAD)                                      \
  do {                                                                       \
    const uint32_t m_ = (VALID) ? (uint32_t)smask[(J)] : 0u;                 \
    const uint32_t bal_ = __ballot_sync(0xffffffffu, m_ != 0);               \
    if (m_) list[n_list + __popc(bal_ & lt)] = make_uint2(m_, (PAYLOAD));    \
    n_list += __popc(bal_);                                                  \
  } while (0)
#define BSX_B16_FLUSH()                                                                        \
  do {                                                                                         \
    __syncwarp();                                                                              \
    if (HETERO && !EAGER) {                                                                    \
      for (int h = lane; h < n_list; h += 32) list[h].y = __float_as_uint(__ldg(rw + list[h].y)); \
      __syncwarp();                                                                            \
    }                                                                                          \
    if (lane == 0 && (n_list & 1)) list[n_list] = make_uint2(0u, 0u);                          \
    __syncwarp();                                                                              \
    const int n_pairs_ = (n_list + 1) >> 1;                                                    \
    for (int h = half; h < n_pairs_; h += 2) {                                                 \
      const uint4 en = pairs[h];                                                               \
      if ((en.x >> b) & 1u) acc += HETERO ? __uint_as_float(en.y) : 1.0f;                      \
      if ((en.z >> b) & 1u) acc += HETERO ? __uint_as_float(en.w) : 1.0f;                      \
    }                                                                                          \
    n_list = 0;                                                                                \
    __syncwarp();                                                                              \
  } while (0)

    // 128-bit body: every lane takes 4 consecutive entries per step
    for (int v0 = 0; v0 < nvec; v0 += 32) {
      const int v = v0 + lane;
      const bool ok = v < nvec;
      int4 j = make_int4(0, 0, 0, 0);
      float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) {
        j = __ldg(r4 + v);
        if (HETERO && EAGER) wv = __ldg(rw4 + v);
      }
      const uint32_t off = (uint32_t)(head + (v << 2));
      BSX_B16_PUSH(ok, j.x, (HETERO && EAGER) ? __float_as_uint(wv.x) : off);
      BSX_B16_PUSH(ok, j.y, (HETERO && EAGER) ? __float_as_uint(wv.y) : off + 1);
      BSX_B16_PUSH(ok, j.z, (HETERO && EAGER) ? __float_as_uint(wv.z) : off + 2);
      BSX_B16_PUSH(ok, j.w, (HETERO && EAGER) ? __float_as_uint(wv.w) : off + 3);
      if (n_list > kB16List - 130) BSX_B16_FLUSH();
    }
    // scalar entries: the head [0, head) and the tail [tail0, len), 32 per step
    const int n_scalar = head + (len - tail0);
    for (int t0 = 0; t0 < n_scalar; t0 += 32) {
      const int t = t0 + lane;
      const bool ok = t < n_scalar;
      const int rel = t < head ? t : tail0 + (t - head);
      const int32_t j = ok ? __ldg(ri + rel) : 0;
      const uint32_t pay = (HETERO && EAGER && ok) ? __float_as_uint(__ldg(rw + rel)) : (uint32_t)rel;
      BSX_B16_PUSH(ok, j, pay);
      if (n_list > kB16List - 130) BSX_B16_FLUSH();
    }
    BSX_B16_FLUSH();
    const float total = acc + __shfl_down_sync(0xffffffffu, acc, 16);
    if (lane < nb) out[(int64_t)lane * n_rows + row] = HETERO ? total : __fmul_rn(total, w0);
#undef BSX_B16_PUSH
#undef BSX_B16_FLUSH
  }
}

// Per warp: phase 1 scans the row and compacts the hits (mask word != 0) into a
// list in shared memory with __ballot_sync/__popc; phase 2 walks the list with
// lane = (half, vector): the lanes of half h take the entry pairs {4k+2h, 4k+2h+1}
// and add the weight of every entry whose bit b is set.  The two halves are
// summed at the end of the row, in a fixed order.
//
// Heterogeneous weights come in two ways, chosen per launch from the measured
// spike density: when more than one synapse in 16 is expected to hit, nearly every
// 32-byte sector of the weight array is needed anyway, so the weights are streamed
// with the indices (128-bit loads); otherwise only the weights of the hits are
// fetched, together, just before the list is walked.
template <bool HETERO>
__global__ void __launch_bounds__(kB16Threads, 1)
event_matvec_b16_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                        const uint16_t* __restrict__ masks, const int32_t* __restrict__ nonzero_words,
                        int64_t n_cols, int64_t n_cols_pad, int64_t n_rows, float* __restrict__ out, int nb,
                        bool vec_ok, bool w_vec_ok, bool use_tma, int weight_mode) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  // [warps][kB16List] hit lists, then the mask words
  uint2* lists = reinterpret_cast<uint2*>(smem_raw);
  uint16_t* smask = reinterpret_cast<uint16_t*>(smem_raw + sizeof(uint2) * kB16List * (kB16Threads / 32));
  stage_bytes(smask, masks, (uint32_t)(n_cols_pad * 2), use_tma, &bar);
  const float w0 = HETERO ? 0.f : __ldg(w);
  // weight_mode: 0 decide from the density, 1 always stream, 2 always fetch on hit
  bool eager = false;
  if (HETERO && w_vec_ok && vec_ok) {
    if (weight_mode == 1) eager = true;
    else if (weight_mode == 0) eager = (int64_t)__ldg(nonzero_words) * 16 > n_cols;
  }
  uint2* list = lists + (threadIdx.x >> 5) * kB16List;
  if (HETERO && eager) b16_rows<HETERO, true>(rm, idx, w, smask, list, n_rows, out, nb, vec_ok, w0);
  else b16_rows<HETERO, false>(rm, idx, w, smask, list, n_rows, out, nb, vec_ok, w0);
}

size_t b16_mask_bytes(int64_t batch, int64_t n_post) {
  const int64_t n_pad = (n_post + 7) & ~int64_t(7);
  const int64_t groups = (batch + kB16 - 1) / kB16;
  // 256 bytes of per-group counters (groups beyond 64 share the last one), then the mask words
  return 256 + (((size_t)groups * (size_t)n_pad * 2 + 255) & ~size_t(255));
}

bool b16_fits(int64_t n_post) {
  const int64_t n_pad = (n_post + 7) & ~int64_t(7);
  return (size_t)n_pad * 2 + sizeof(uint2) * kB16List * (kB16Threads / 32) <= 200 * 1024;
}

// spikes: (batch, n_post) in `format` (BOOL8, F32 or BITS32).  masks: workspace of
// b16_mask_bytes.  out: (batch, n_pre).
int launch_event_matvec_b16(const bsx_conn_t* conn, const void* spikes, int format, int64_t batch, float* out,
                            void* workspace, int weight_mode, cudaStream_t st) {
  const int64_t n_post = conn->n_post, n_pre = conn->n_pre;
  const int64_t n_pad = (n_post + 7) & ~int64_t(7);
  const int64_t groups = (batch + kB16 - 1) / kB16;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  if (groups > 64) return fail(BSX_ERR_UNSUPPORTED, "batched event matvec takes at most 1024 vectors per call");
  int32_t* counters = static_cast<int32_t*>(workspace);
  uint16_t* m16 = reinterpret_cast<uint16_t*>(static_cast<char*>(workspace) + 256);
  void* masks = m16;
  BSX_CUDA(cudaMemsetAsync(counters, 0, 256, st));
  {
    int64_t total = groups * n_pad;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    if (format == BSX_SPK_BOOL8)
      pack16_kernel<BSX_SPK_BOOL8><<<(unsigned)blocks, 256, 0, st>>>(spikes, batch, n_post, n_pad, m16, counters);
    else if (format == BSX_SPK_F32)
      pack16_kernel<BSX_SPK_F32><<<(unsigned)blocks, 256, 0, st>>>(spikes, batch, n_post, n_pad, m16, counters);
    else if (format == BSX_SPK_BITS32)
      pack16_kernel<BSX_SPK_BITS32><<<(unsigned)blocks, 256, 0, st>>>(spikes, batch, n_post, n_pad, m16, counters);
    else
      return fail(BSX_ERR_INVALID_ARG, "batched event matvec takes BOOL8, F32 or BITS32 spikes");
    BSX_LAUNCH_CHECK("pack16_kernel");
  }
  const size_t smem = (size_t)n_pad * 2 + sizeof(uint2) * kB16List * (kB16Threads / 32);
  const bool vec_ok = aligned16(conn->indices);
  const bool w_vec_ok = conn->hetero && aligned16(conn->weights);
  const bool use_tma = aligned16(masks) && ((n_pad * 2) % 16 == 0);
  const RowMap rm = make_rowmap(conn);
  int64_t blocks = (n_pre + (kB16Threads / 32) - 1) / (kB16Threads / 32);
  if (blocks > sms) blocks = sms;
  if (blocks < 1) blocks = 1;
  if (conn->hetero)
    BSX_CUDA(cudaFuncSetAttribute(event_matvec_b16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  else
    BSX_CUDA(cudaFuncSetAttribute(event_matvec_b16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  for (int64_t g = 0; g < groups; ++g) {
    const int nb = (int)((batch - g * kB16) < kB16 ? (batch - g * kB16) : kB16);
    float* og = out + g * kB16 * n_pre;
    const uint16_t* mg = m16 + g * n_pad;
    if (conn->hetero)
      event_matvec_b16_kernel<true><<<(unsigned)blocks, kB16Threads, smem, st>>>(
          rm, conn->indices, conn->weights, mg, counters + g, n_post, n_pad, n_pre, og, nb, vec_ok, w_vec_ok,
          use_tma, weight_mode);
    else
      event_matvec_b16_kernel<false><<<(unsigned)blocks, kB16Threads, smem, st>>>(
          rm, conn->indices, conn->weights, mg, counters + g, n_post, n_pad, n_pre, og, nb, vec_ok, w_vec_ok,
          use_tma, weight_mode);
    BSX_LAUNCH_CHECK("event_matvec_b16_kernel");
  }
  return BSX_OK;
}

}  // namespace bsx
