// Event vecmat for one (or a few) spike vectors in ONE kernel launch.
//
// This is the call EventFixedProb.update(spk) makes once per simulation step
// (brainstate/nn/_event_fixedprob.py:202-205,249-252): a single spike vector, a few
// hundred active rows.  Queueing the active rows in global memory, clearing the output and
// scattering as dependent launches costs more in launch latency than in memory traffic.
// Here the output is cleared by a memset node on the stream and ONE kernel does the rest:
//
//   1. every block scans the WHOLE spike vector (at most 128 KB, served by L2) and builds
//      the complete list of active rows in its own shared memory — the same list in every
//      block, so no queue in global memory, no atomic counter and no second kernel;
//   2. the warps of all blocks share the (active row, chunk) items round-robin and scatter
//      them with red.global.add.f32.
//
// Blocks never wait for one another.  A list input (BSX_SPK_LIST) is read in place.
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

constexpr int kFuThreads = 1024;
constexpr int kFuWarps = kFuThreads / 32;
constexpr int kFuLoads = 8;                                  // 16-byte loads per thread
constexpr int64_t kFuBytes = (int64_t)kFuThreads * kFuLoads * 16;   // spike bytes one call may scan
constexpr int kFuList = 8192;                                // active rows staged per round

// 16 spike bytes / 4 floats / 4 packed words starting at byte `off`; bytes past `nbytes` read as zero.
__device__ __forceinline__ uint4 load_chunk(const unsigned char* __restrict__ p, int64_t off, int64_t nbytes) {
  if (off + 16 <= nbytes) return __ldg(reinterpret_cast<const uint4*>(p + off));
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  for (int k = 0; k < 16 && off + k < nbytes; ++k) w[k >> 2] |= (uint32_t)p[off + k] << (8 * (k & 3));
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// bit k: byte k of v is nonzero.  One SIMD compare gives 0x01 per nonzero byte; the multiplication
// adds byte i shifted to bit i of the top byte (1*b0 + 2*b1 + 4*b2 + 8*b3; no carries: at most 15).
__device__ __forceinline__ uint32_t byte_flags(uint32_t v) {
  return ((__vcmpne4(v, 0u) & 0x01010101u) * 0x01020408u) >> 24;
}

// Active spikes of one chunk as up to four (mask, flat index of bit 0) pairs.
template <int FORMAT>
__device__ __forceinline__ void chunk_masks(const uint4& v, int64_t chunk, int64_t n_pre, int64_t words,
                                            uint32_t m[4], int64_t base[4]) {
  const uint32_t raw[4] = {v.x, v.y, v.z, v.w};
  if (FORMAT == BSX_SPK_BOOL8) {
    m[0] = byte_flags(raw[0]) | (byte_flags(raw[1]) << 4) | (byte_flags(raw[2]) << 8) | (byte_flags(raw[3]) << 12);
    base[0] = chunk * 16;
    m[1] = m[2] = m[3] = 0;
    base[1] = base[2] = base[3] = 0;
  } else if (FORMAT == BSX_SPK_F32) {
    // +0.0f and -0.0f are both "no spike"
    m[0] = ((raw[0] << 1) ? 1u : 0u) | ((raw[1] << 1) ? 2u : 0u) | ((raw[2] << 1) ? 4u : 0u) | ((raw[3] << 1) ? 8u : 0u);
    base[0] = chunk * 4;
    m[1] = m[2] = m[3] = 0;
    base[1] = base[2] = base[3] = 0;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t g = chunk * 4 + j;                       // word index over all batch rows
      const int64_t b = g / words, wi = g - b * words;
      const int64_t left = n_pre - wi * 32;                  // valid bits of this word
      m[j] = raw[j] & (left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << left) - 1u)));
      base[j] = b * n_pre + wi * 32;
    }
  }
}

// The thread's kFuLoads chunks (chunk j * kFuThreads + tid), all loads issued before any is used:
// one round trip to L2 instead of one per chunk.  Whole chunks are plain 128-bit loads; only the
// last, partial chunk of the input goes through the byte-wise loader.
__device__ __forceinline__ void load_my_chunks(const unsigned char* __restrict__ spikes, int64_t spike_bytes, int tid,
                                               uint4 v[kFuLoads]) {
  const int64_t whole = spike_bytes >> 4;
  const uint4* __restrict__ p4 = reinterpret_cast<const uint4*>(spikes);
#pragma unroll
  for (int j = 0; j < kFuLoads; ++j) {
    const int64_t c = (int64_t)j * kFuThreads + tid;
    v[j] = c < whole ? __ldg(p4 + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  if (spike_bytes & 15) {
    const int64_t c = whole;                                  // the partial chunk
    const int j = (int)(c / kFuThreads);
    if (c - (int64_t)j * kFuThreads == tid && j < kFuLoads) {
      const uint4 t = load_chunk(spikes, c * 16, spike_bytes);
#pragma unroll
      for (int k = 0; k < kFuLoads; ++k)
        if (k == j) v[k] = t;
    }
  }
}

template <bool HETERO, bool HAS_X, int FORMAT>
__global__ void __launch_bounds__(kFuThreads, 1)
scatter_fused_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                     const unsigned char* __restrict__ spikes, int64_t spike_bytes, const float* __restrict__ x,
                     float* __restrict__ out, int64_t n_pre, int64_t n_post, int64_t batch, int chunks_per_row,
                     int chunk, bool vec_ok, float* __restrict__ clear_next = nullptr, int64_t clear_count = 0) {
  __shared__ uint32_t s_list[kFuList];
  __shared__ uint32_t s_warp[kFuWarps];
  __shared__ uint32_t s_total;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int64_t gwarp = (int64_t)blockIdx.x * kFuWarps + wid;
  const int64_t gwarps = (int64_t)gridDim.x * kFuWarps;
  // ---- 0. a caller that alternates between output buffers has this launch clear the one the
  // next launch adds into, which saves the separate clearing node of every call
  if (clear_next) {
    const int64_t gt = (int64_t)blockIdx.x * kFuThreads + tid, gn = (int64_t)gridDim.x * kFuThreads;
    if ((reinterpret_cast<uintptr_t>(clear_next) & 15) == 0) {
      float4* c4 = reinterpret_cast<float4*>(clear_next);
      for (int64_t i = gt; i < (clear_count >> 2); i += gn) c4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int64_t i = (clear_count & ~int64_t(3)) + gt; i < clear_count; i += gn) clear_next[i] = 0.f;
    } else {
      for (int64_t i = gt; i < clear_count; i += gn) clear_next[i] = 0.f;
    }
  }
  // ---- 1. the list of active rows (every block builds the same one) ----
  const uint32_t* entries = s_list;
  uint32_t total = 0;
  uint32_t my_off = 0;
  const int64_t words = (n_pre + 31) >> 5;
  // byte and float inputs: a chunk's spikes are one mask of 16 or 4 bits, kept in a register from
  // the count pass to the list pass (packed words are four masks per chunk: they are read again)
  constexpr bool KEEP = FORMAT == BSX_SPK_BOOL8 || FORMAT == BSX_SPK_F32;
  uint32_t mk[kFuLoads];
  if (FORMAT == BSX_SPK_LIST) {
    const int32_t* list = reinterpret_cast<const int32_t*>(spikes);
    total = (uint32_t)__ldg(list);
    entries = reinterpret_cast<const uint32_t*>(list + 1);
  } else {
    uint32_t cnt = 0;
    uint4 v[kFuLoads];
    load_my_chunks(spikes, spike_bytes, tid, v);
#pragma unroll
    for (int j = 0; j < kFuLoads; ++j) {
      const int64_t c = (int64_t)j * kFuThreads + tid;
      mk[j] = 0;
      if (c * 16 < spike_bytes) {
        uint32_t m[4];
        int64_t base[4];
        chunk_masks<FORMAT>(v[j], c, n_pre, words, m, base);
        cnt += __popc(m[0]) + __popc(m[1]) + __popc(m[2]) + __popc(m[3]);
        if (KEEP) mk[j] = m[0];
      }
    }
    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      uint32_t v = s_warp[lane], inc = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      s_warp[lane] = inc - v;
      if (lane == 31) s_total = inc;
    }
    __syncthreads();
    my_off = s_warp[wid] + incl - cnt;
    total = s_total;
  }
  // ---- 2. scatter, in rounds of kFuList rows when the list is longer than shared memory ----
  // Few active rows: small chunks spread each row over many warps (latency).  Many:
  // eight times larger chunks, fewer and longer streams per warp (throughput).
  if (chunks_per_row > 1 && (int64_t)total * chunks_per_row > 4 * gwarps) {
    chunk *= 8;
    chunks_per_row = (chunks_per_row + 7) >> 3;
  }
  const float w0 = HETERO ? 1.0f : __ldg(w);
  const uint32_t rounds = FORMAT == BSX_SPK_LIST ? 1u : (total + kFuList - 1) / kFuList;
  for (uint32_t r = 0; r < rounds; ++r) {
    uint32_t r_count = total;
    if (FORMAT != BSX_SPK_LIST) {
      const uint32_t lo = r * kFuList;
      r_count = total - lo < (uint32_t)kFuList ? total - lo : (uint32_t)kFuList;
      if (r > 0) __syncthreads();                             // the previous round's list has been consumed
      uint32_t pos = my_off;
      uint4 v[kFuLoads];
      if (!KEEP) load_my_chunks(spikes, spike_bytes, tid, v);   // L1/L2 hits: the count pass just read them
#pragma unroll
      for (int j = 0; j < kFuLoads; ++j) {
        const int64_t c = (int64_t)j * kFuThreads + tid;
        if (c * 16 < spike_bytes) {
          uint32_t m[4];
          int64_t base[4];
          if (KEEP) {
            m[0] = mk[j];
            base[0] = c * (FORMAT == BSX_SPK_BOOL8 ? 16 : 4);
            m[1] = m[2] = m[3] = 0;
            base[1] = base[2] = base[3] = 0;
          } else {
            chunk_masks<FORMAT>(v[j], c, n_pre, words, m, base);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t mm = m[u];
            while (mm) {
              const int k = __ffs(mm) - 1;
              mm &= mm - 1;
              const uint32_t at = pos - lo;                   // wraps to a large value below lo
              if (at < (uint32_t)kFuList) s_list[at] = (uint32_t)(base[u] + k);
              ++pos;
            }
          }
        }
      }
      __syncthreads();
    }
    const int64_t items = (int64_t)r_count * chunks_per_row;
    for (int64_t it = gwarp; it < items; it += gwarps) {
      const int64_t q = it / chunks_per_row;
      const int c = (int)(it - q * chunks_per_row);
      const uint32_t flat = entries[q];
      int64_t b = 0, i = flat;
      if (batch > 1) {
        b = flat / n_pre;
        i = flat - b * n_pre;
      }
      int64_t s, e;
      rm.range(i, s, e);
      if (chunks_per_row > 1) {
        s += (int64_t)c * chunk;
        if (s >= e) continue;
        if (s + chunk < e) e = s + chunk;
      }
      float v = HAS_X ? __ldg(x + flat) : 1.0f;
      if (!HETERO) v = __fmul_rn(v, w0);
      scatter_span<HETERO>(idx, w, s, e, lane, v, out + b * n_post, vec_ok);
    }
  }
}

// The spike input is small enough for every block to scan all of it.
bool scatter_fused_fits(const bsx_conn_t* conn, int format, int64_t batch) {
  if (conn->indptr == nullptr && conn->conn_num == 0) return false;
  if (format == BSX_SPK_LIST) return batch == 1;
  const int64_t n = batch * conn->n_pre;
  const int64_t bytes = format == BSX_SPK_BOOL8 ? n : format == BSX_SPK_F32 ? 4 * n : 4 * batch * ((conn->n_pre + 31) / 32);
  return bytes <= kFuBytes;
}

bool scatter_fused_applies(const bsx_conn_t* conn, const void* spikes, int format, int64_t batch) {
  if (!scatter_fused_fits(conn, format, batch)) return false;
  return format == BSX_SPK_LIST ? (reinterpret_cast<uintptr_t>(spikes) & 3) == 0 : aligned16(spikes);
}

int launch_scatter_fused(const bsx_conn_t* conn, const void* spikes, int format, const float* x, int64_t batch,
                         float* out, int accumulate, cudaStream_t st, float* clear_next) {
  const int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int chunk = 128, cpr = 1;
  if (!conn->indptr && conn->conn_num > chunk) {
    int64_t c = (conn->conn_num + chunk - 1) / chunk;
    if (c > 1 << 20) {
      chunk = (int)((conn->conn_num + (1 << 20) - 1) >> 20);
      c = (conn->conn_num + chunk - 1) / chunk;
    }
    cpr = (int)c;
  }
  const bool vec_ok = aligned16(conn->indices) && (!conn->hetero || aligned16(conn->weights));
  const RowMap rm = make_rowmap(conn);
  const int64_t n = batch * conn->n_pre;
  const int64_t spike_bytes = format == BSX_SPK_BOOL8 ? n : format == BSX_SPK_F32 ? 4 * n
                              : format == BSX_SPK_BITS32 ? 4 * batch * ((conn->n_pre + 31) / 32) : 0;
  if (!accumulate)
    BSX_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)batch * (size_t)conn->n_post, st));
  const unsigned char* sp = static_cast<const unsigned char*>(spikes);
  const unsigned grid = (unsigned)sms;
#define BSX_FUSED(H, X, F)                                                                                       \
  scatter_fused_kernel<H, X, F><<<grid, kFuThreads, 0, st>>>(rm, conn->indices, conn->weights, sp, spike_bytes, x, out, \
                                                             conn->n_pre, conn->n_post, batch, cpr, chunk, vec_ok, \
                                                             clear_next, clear_next ? batch * conn->n_post : 0)
#define BSX_FUSED_FMT(H, X)                                        \
  switch (format) {                                                \
    case BSX_SPK_BOOL8: BSX_FUSED(H, X, BSX_SPK_BOOL8); break;     \
    case BSX_SPK_F32: BSX_FUSED(H, X, BSX_SPK_F32); break;         \
    case BSX_SPK_BITS32: BSX_FUSED(H, X, BSX_SPK_BITS32); break;   \
    default: BSX_FUSED(H, X, BSX_SPK_LIST); break;                 \
  }
  if (conn->hetero) {
    if (x) { BSX_FUSED_FMT(true, true) } else { BSX_FUSED_FMT(true, false) }
  } else {
    if (x) { BSX_FUSED_FMT(false, true) } else { BSX_FUSED_FMT(false, false) }
  }
#undef BSX_FUSED_FMT
#undef BSX_FUSED
  BSX_LAUNCH_CHECK("scatter_fused_kernel");
  return BSX_OK;
}

}  // namespace bsx
