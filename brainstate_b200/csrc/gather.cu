// Row-gather products: one warp per matrix row, no atomics, fixed summation
// order (lane-strided partial sums, then a butterfly), hence deterministic.
//
//   event matvec   y[i] = sum_k w[i,k] * [s[idx[i,k]] != 0]    spike bits in shared memory
//   float matvec   y[i] = sum_k w[i,k] * v[idx[i,k]]           v read through L2
//   vecmat vjp     dx (= float matvec of ct) and dw in one pass over the indices
//
// HBM traffic: 4 B per stored synapse for the indices; weights are touched only
// where a spike hits (event) or for every synapse (float / vjp).
#include "bsx_tuning.h"
#include "bulk_copy.cuh"
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

// Copies `words` 32-bit words into shared memory.  With use_tma the copy is one
// or more bulk-async transfers completing on an mbarrier; every wait is bounded
// and, should it run out, the block re-reads the words with ordinary loads (the
// data are identical, so a late transfer is harmless).
__device__ __forceinline__ void stage_words(uint32_t* __restrict__ smem, const uint32_t* __restrict__ gmem,
                                            int64_t words, bool use_tma, uint64_t* bar) {
  bool done = false;
  if (use_tma) {
    const uint32_t bytes = (uint32_t)(words * 4);
    if (threadIdx.x == 0) mbar_init(bar, 1);
    __syncthreads();
    if (threadIdx.x == 0) {
      mbar_expect_tx(bar, bytes);
      const uint32_t piece = 32768;
      for (uint32_t off = 0; off < bytes; off += piece) {
        const uint32_t sz = bytes - off < piece ? bytes - off : piece;
        bulk_g2s(reinterpret_cast<char*>(smem) + off, reinterpret_cast<const char*>(gmem) + off, sz, bar);
      }
    }
    bool ok = false;
    for (int spin = 0; spin < (1 << 22) && !ok; ++spin) ok = mbar_try_wait(bar, 0);
    done = __syncthreads_and(ok);
  }
  if (!done) {
    for (int64_t i = threadIdx.x; i < words; i += blockDim.x) smem[i] = __ldg(gmem + i);
    __syncthreads();
  }
}

__device__ __forceinline__ bool bit_at(const uint32_t* __restrict__ m, int32_t j) {
  return (m[j >> 5] >> (j & 31)) & 1u;
}

// ---- event matvec -------------------------------------------------------------
// U = number of 128-bit index loads each lane issues before it consumes any of
// them.  A 655-entry row is 164 such loads, i.e. 6 per lane: with U = 6 a warp has
// its whole row in flight at once.
template <bool HETERO, bool SMEM, int U>
__global__ void __launch_bounds__(256, (U > 2 ? 4 : (U > 1 ? 6 : 8)))
event_matvec_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                    const uint32_t* __restrict__ bits, int64_t words, int64_t n_rows,
                    float* __restrict__ out, bool vec_ok, bool use_tma) {
  extern __shared__ __align__(16) uint32_t smask[];
  __shared__ __align__(8) uint64_t bar;
  const int lane = threadIdx.x & 31;
  const int64_t b = blockIdx.y;
  const uint32_t* __restrict__ gbits = bits + b * words;
  const uint32_t* __restrict__ mask = gbits;
  if (SMEM) {
    stage_words(smask, gbits, words, use_tma, &bar);
    mask = smask;
  }
  float* __restrict__ ob = out + b * n_rows;
  const float w0 = HETERO ? 0.f : __ldg(w);
  const int4* __restrict__ idx4 = reinterpret_cast<const int4*>(idx);
  const int64_t wstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += wstep) {
    int64_t s, e;
    rm.range(row, s, e);
    float acc = 0.f;
    int hits = 0;
    int64_t a0 = e, a1 = e;  // no vector body unless aligned
    if (vec_ok) {
      a0 = (s + 3) & ~int64_t(3);
      if (a0 > e) a0 = e;
      a1 = e & ~int64_t(3);
      if (a1 < a0) a1 = a0;
    }
    const int64_t q1 = a1 >> 2;
    for (int64_t qb = (a0 >> 2) + lane; qb < q1 + lane; qb += 32 * U) {
      int4 j[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t q = qb + 32 * u;
        if (q < q1) j[u] = __ldg(idx4 + q);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t q = qb + 32 * u;
        if (q < q1) {
          const bool h0 = bit_at(mask, j[u].x), h1 = bit_at(mask, j[u].y), h2 = bit_at(mask, j[u].z),
                     h3 = bit_at(mask, j[u].w);
          if (HETERO) {
            const float* wp = w + (q << 2);
            if (h0) acc += __ldg(wp);
            if (h1) acc += __ldg(wp + 1);
            if (h2) acc += __ldg(wp + 2);
            if (h3) acc += __ldg(wp + 3);
          } else {
            hits += (int)h0 + (int)h1 + (int)h2 + (int)h3;
          }
        }
      }
    }
    // scalar head [s, a0) and tail [a1, e)
    for (int64_t p = s + lane; p < a0; p += 32)
      if (bit_at(mask, __ldg(idx + p))) {
        if (HETERO) acc += __ldg(w + p); else ++hits;
      }
    for (int64_t p = a1 + lane; p < e; p += 32)
      if (bit_at(mask, __ldg(idx + p))) {
        if (HETERO) acc += __ldg(w + p); else ++hits;
      }
    if (HETERO) {
      acc = warp_sum(acc);
    } else {
      hits = __reduce_add_sync(0xffffffffu, hits);
      acc = __fmul_rn((float)hits, w0);
    }
    if (lane == 0) ob[row] = acc;
  }
}

// ---- float matvec ---------------------------------------------------------------
template <bool HETERO>
__global__ void __launch_bounds__(256)
float_matvec_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                    const float* __restrict__ v, int64_t n_cols, int64_t n_rows, float* __restrict__ out,
                    bool vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t b = blockIdx.y;
  const float* __restrict__ vb = v + b * n_cols;
  float* __restrict__ ob = out + b * n_rows;
  const float w0 = HETERO ? 0.f : __ldg(w);
  const int4* __restrict__ idx4 = reinterpret_cast<const int4*>(idx);
  const float4* __restrict__ w4 = reinterpret_cast<const float4*>(w);
  const int64_t wstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += wstep) {
    int64_t s, e;
    rm.range(row, s, e);
    float acc = 0.f;
    int64_t a0 = e, a1 = e;  // no vector body unless aligned
    if (vec_ok) {
      a0 = (s + 3) & ~int64_t(3);
      if (a0 > e) a0 = e;
      a1 = e & ~int64_t(3);
      if (a1 < a0) a1 = a0;
    }
    for (int64_t p = s + lane; p < a0; p += 32) acc += __ldg(vb + __ldg(idx + p)) * (HETERO ? __ldg(w + p) : 1.f);
    for (int64_t p = a1 + lane; p < e; p += 32) acc += __ldg(vb + __ldg(idx + p)) * (HETERO ? __ldg(w + p) : 1.f);
    const int64_t q1 = a1 >> 2;
#pragma unroll 2
    for (int64_t q = (a0 >> 2) + lane; q < q1; q += 32) {
      const int4 j = __ldg(idx4 + q);
      const float c0 = __ldg(vb + j.x), c1 = __ldg(vb + j.y), c2 = __ldg(vb + j.z), c3 = __ldg(vb + j.w);
      if (HETERO) {
        const float4 ww = __ldg(w4 + q);
        acc += c0 * ww.x;
        acc += c1 * ww.y;
        acc += c2 * ww.z;
        acc += c3 * ww.w;
      } else {
        acc += (c0 + c1) + (c2 + c3);
      }
    }
    acc = warp_sum(acc);
    if (!HETERO) acc *= w0;
    if (lane == 0) ob[row] = acc;
  }
}

// ---- reverse mode: dx and dw in one pass ---------------------------------------
// DW_MODE 0: no dw; 1: dw[p] = a*c written for every row (batch 1);
// 2: dw pre-zeroed, rows with a != 0 add a*c (red for batch > 1); 3: homogeneous scalar.
template <bool HETERO, int DW_MODE, int XFORMAT>
__global__ void __launch_bounds__(256)
vjp_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w, const void* __restrict__ x,
           bool event, const float* __restrict__ ct, int64_t n_pre, int64_t n_post, float* __restrict__ dx,
           float* __restrict__ dw, bool atomic_dw) {
  __shared__ float block_part[8];
  const int lane = threadIdx.x & 31;
  const int64_t b = blockIdx.y;
  const float* __restrict__ cb = ct + b * n_post;
  const float w0 = HETERO ? 0.f : __ldg(w);
  float homo_acc = 0.f;
  const int64_t wstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_pre; row += wstep) {
    float a = 0.f;
    if (DW_MODE != 0) {
      a = (XFORMAT == BSX_SPK_BOOL8) ? (float)(static_cast<const uint8_t*>(x)[b * n_pre + row] != 0)
                                     : static_cast<const float*>(x)[b * n_pre + row];
      if (event) a = (a != 0.f) ? 1.f : 0.f;
    }
    if (!dx && (DW_MODE == 2 || DW_MODE == 3) && a == 0.f) continue;  // nothing to produce for this row
    int64_t s, e;
    rm.range(row, s, e);
    float acc = 0.f, csum = 0.f;
    for (int64_t p = s + lane; p < e; p += 32) {
      const float c = __ldg(cb + __ldg(idx + p));
      if (HETERO) acc += c * __ldg(w + p); else csum += c;
      if (DW_MODE == 1) dw[p] = __fmul_rn(a, c);
      if (DW_MODE == 2 && a != 0.f) {
        if (atomic_dw) red_add(dw + p, __fmul_rn(a, c)); else dw[p] = __fmul_rn(a, c);
      }
    }
    if (!HETERO) acc = csum;
    acc = warp_sum(acc);
    if (!HETERO) {
      if (DW_MODE == 3) homo_acc += a * acc;  // acc is still the plain sum of ct here
      acc *= w0;
    }
    if (dx && lane == 0) dx[b * n_pre + row] = acc;
  }
  if (DW_MODE == 3) {
    if (lane == 0) block_part[threadIdx.x >> 5] = homo_acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += block_part[k];
      if (t != 0.f) red_add(dw, t);
    }
  }
}

static int row_grid(int64_t n_rows, int64_t batch, int blocks_per_sm, dim3* grid) {
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  if (batch > 65535) return fail(BSX_ERR_UNSUPPORTED, "batch above 65535");
  int64_t blocks = (n_rows + 7) / 8;
  int64_t cap = (int64_t)sms * blocks_per_sm;
  if (batch > 1) cap = (cap + batch - 1) / batch < sms ? sms : (cap + batch - 1) / batch;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  *grid = dim3((unsigned)blocks, (unsigned)batch, 1);
  return BSX_OK;
}

}  // namespace bsx

using namespace bsx;

extern "C" {

static size_t packed_words_bytes(int64_t batch, int64_t n_post) {
  size_t b = sizeof(uint32_t) * (size_t)batch * (size_t)((n_post + 31) / 32);
  return (b + 255) & ~size_t(255);
}

size_t bsx_event_matvec_workspace_bytes(int64_t batch, int64_t n_post) {
  if (batch < 0 || n_post < 0) return 0;
  const size_t a = packed_words_bytes(batch, n_post);
  const size_t b = (batch >= 2 && b16_fits(n_post)) ? b16_mask_bytes(batch, n_post) : 0;
  return a > b ? a : b;
}

int bsx_event_matvec_tuned(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                           float* out, void* workspace, size_t workspace_bytes, int blocks_per_sm,
                           int mask_mode, int unroll, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_matvec_tuned");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (batch == 0 || conn->n_pre == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  cudaStream_t st = as_stream(stream);
  const bool empty = !conn->indptr && conn->conn_num == 0;
  if (empty || conn->n_post == 0) return launch_zero(out, batch * conn->n_pre, st);
  if (!spikes) return fail(BSX_ERR_INVALID_ARG, "spikes is NULL");
  if (spike_format != BSX_SPK_BITS32 && spike_format != BSX_SPK_BOOL8 && spike_format != BSX_SPK_F32)
    return fail(BSX_ERR_INVALID_ARG, "event matvec takes BOOL8, F32 or BITS32 spikes");
  // two or more vectors: one pass over the indices serves 16 vectors (mask_mode 4 opts out)
  if (batch >= 2 && mask_mode != 4 && b16_fits(conn->n_post) && workspace &&
      (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 &&
      workspace_bytes >= b16_mask_bytes(batch, conn->n_post))
    return launch_event_matvec_b16(conn, spikes, spike_format, batch, out, workspace,
                                   mask_mode == 5 ? 1 : (mask_mode == 6 ? 2 : 0), st);
  const int64_t words = (conn->n_post + 31) / 32;
  const uint32_t* bits;
  if (spike_format == BSX_SPK_BITS32) {
    bits = static_cast<const uint32_t*>(spikes);
  } else if (spike_format == BSX_SPK_BOOL8 || spike_format == BSX_SPK_F32) {
    if (!workspace || workspace_bytes < packed_words_bytes(batch, conn->n_post))
      return fail(BSX_ERR_WORKSPACE, "event matvec needs %zu workspace bytes for the packed spikes",
                  packed_words_bytes(batch, conn->n_post));
    rc = launch_pack(spikes, spike_format, batch, conn->n_post, static_cast<uint32_t*>(workspace), st);
    if (rc) return rc;
    bits = static_cast<const uint32_t*>(workspace);
  } else {
    return fail(BSX_ERR_INVALID_ARG, "event matvec takes BOOL8, F32 or BITS32 spikes");
  }
  if (unroll != 1 && unroll != 2 && unroll != 4 && unroll != 6) unroll = 6;
  if (blocks_per_sm <= 0) blocks_per_sm = unroll > 2 ? 4 : 8;
  dim3 grid;
  rc = row_grid(conn->n_pre, batch, blocks_per_sm, &grid);
  if (rc) return rc;
  // mask_mode: 0 auto, 1 shared memory + bulk-async copy, 2 shared memory + plain loads, 3 global
  const size_t smem = (size_t)words * 4;
  // keep 8 resident blocks per SM when the words are few; large masks trade occupancy for locality
  bool use_smem = smem <= 200 * 1024;
  if (mask_mode == 3) use_smem = false;
  const bool tma_ok = aligned16(bits) && (words % 4 == 0) && smem < (1u << 20);
  const bool use_tma = use_smem && tma_ok && mask_mode != 2;
  const bool vec_ok = aligned16(conn->indices);
  const RowMap rm = make_rowmap(conn);
#define BSX_EMV_U(H, S, SM, UU)                                                                  \
  do {                                                                                          \
    if ((SM) > 48 * 1024)                                                                       \
      BSX_CUDA(cudaFuncSetAttribute(event_matvec_kernel<H, S, UU>,                               \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SM)));    \
    event_matvec_kernel<H, S, UU><<<grid, 256, (SM), st>>>(rm, conn->indices, conn->weights, bits, \
                                                           words, conn->n_pre, out, vec_ok, use_tma); \
  } while (0)
#define BSX_EMV(H, S, SM)                        \
  do {                                           \
    if (unroll == 1) BSX_EMV_U(H, S, SM, 1);     \
    else if (unroll == 2) BSX_EMV_U(H, S, SM, 2); \
    else if (unroll == 4) BSX_EMV_U(H, S, SM, 4); \
    else BSX_EMV_U(H, S, SM, 6);                 \
  } while (0)
  if (use_smem) {
    if (smem > 24 * 1024) {  // fewer, fatter blocks: one mask copy per resident block
      int per_sm = (int)((200 * 1024) / smem);
      if (per_sm < 1) per_sm = 1;
      if (per_sm < blocks_per_sm) {
        rc = row_grid(conn->n_pre, batch, per_sm, &grid);
        if (rc) return rc;
      }
    }
    if (conn->hetero) BSX_EMV(true, true, smem); else BSX_EMV(false, true, smem);
  } else {
    if (conn->hetero) BSX_EMV(true, false, 0); else BSX_EMV(false, false, 0);
  }
#undef BSX_EMV
#undef BSX_EMV_U
  BSX_LAUNCH_CHECK("event_matvec_kernel");
  return BSX_OK;
}

int bsx_event_matvec(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                     float* out, void* workspace, size_t workspace_bytes, bsx_stream_t stream) {
  return bsx_event_matvec_tuned(conn, spikes, spike_format, batch, out, workspace, workspace_bytes, 0, 0, 0,
                                stream);
}

int bsx_float_matvec(const bsx_conn_t* conn, const float* v, int64_t batch, float* out, bsx_stream_t stream) {
  BSX_TRACE("bsx_float_matvec");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (batch == 0 || conn->n_pre == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  cudaStream_t st = as_stream(stream);
  const bool empty = !conn->indptr && conn->conn_num == 0;
  if (empty || conn->n_post == 0) return launch_zero(out, batch * conn->n_pre, st);
  if (!v) return fail(BSX_ERR_INVALID_ARG, "v is NULL");
  dim3 grid;
  rc = row_grid(conn->n_pre, batch, 8, &grid);
  if (rc) return rc;
  const bool vec_ok = aligned16(conn->indices) && (!conn->hetero || aligned16(conn->weights));
  const RowMap rm = make_rowmap(conn);
  if (conn->hetero)
    float_matvec_kernel<true><<<grid, 256, 0, st>>>(rm, conn->indices, conn->weights, v, conn->n_post,
                                                    conn->n_pre, out, vec_ok);
  else
    float_matvec_kernel<false><<<grid, 256, 0, st>>>(rm, conn->indices, conn->weights, v, conn->n_post,
                                                     conn->n_pre, out, vec_ok);
  BSX_LAUNCH_CHECK("float_matvec_kernel");
  return BSX_OK;
}

int bsx_vecmat_vjp(const bsx_conn_t* conn, const void* x, int x_format, int event, const float* ct,
                   int64_t batch, float* dx, float* dw, bsx_stream_t stream) {
  BSX_TRACE("bsx_vecmat_vjp");
  int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (x_format != BSX_SPK_BOOL8 && x_format != BSX_SPK_F32)
    return fail(BSX_ERR_INVALID_ARG, "vjp takes the primal input as BOOL8 or F32");
  cudaStream_t st = as_stream(stream);
  const bool empty = conn->n_pre == 0 || (!conn->indptr && conn->conn_num == 0) || conn->n_post == 0;
  if (dw && !conn->hetero) {
    rc = launch_zero(dw, 1, st);
    if (rc) return rc;
  }
  if (batch == 0 || empty) {
    if (dx && batch > 0 && conn->n_pre > 0) return launch_zero(dx, batch * conn->n_pre, st);
    return BSX_OK;
  }
  if (!ct) return fail(BSX_ERR_INVALID_ARG, "ct is NULL");
  if (dw && !x) return fail(BSX_ERR_INVALID_ARG, "the weight cotangent needs the primal input x");
  if (!dx && !dw) return BSX_OK;
  dim3 grid;
  rc = row_grid(conn->n_pre, batch, 8, &grid);
  if (rc) return rc;
  const RowMap rm = make_rowmap(conn);
  int mode = 0;
  bool atomic_dw = false;
  if (dw && !conn->hetero) mode = 3;
  else if (dw && batch == 1 && dx) mode = 1;
  else if (dw) {
    mode = 2;
    atomic_dw = batch > 1;
    rc = launch_zero(dw, conn->nnz, st);
    if (rc) return rc;
  }
  const bool ev = event != 0;
#define BSX_VJP(H, M, F)                                                                               \
  vjp_kernel<H, M, F><<<grid, 256, 0, st>>>(rm, conn->indices, conn->weights, x, ev, ct, conn->n_pre,  \
                                            conn->n_post, dx, dw, atomic_dw)
#define BSX_VJP_F(H, M)                                                   \
  do {                                                                    \
    if (x_format == BSX_SPK_BOOL8) BSX_VJP(H, M, BSX_SPK_BOOL8);          \
    else BSX_VJP(H, M, BSX_SPK_F32);                                      \
  } while (0)
  if (conn->hetero) {
    if (mode == 0) BSX_VJP_F(true, 0);
    else if (mode == 1) BSX_VJP_F(true, 1);
    else BSX_VJP_F(true, 2);
  } else {
    if (mode == 0) BSX_VJP_F(false, 0);
    else BSX_VJP_F(false, 3);
  }
#undef BSX_VJP_F
#undef BSX_VJP
  BSX_LAUNCH_CHECK("vjp_kernel");
  return BSX_OK;
}

}  // extern "C"
