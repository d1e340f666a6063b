// Pre-centric scatter: y[b, idx[i,k]] += a[b,i] * w[i,k] for every active (b, i).
//
// Stage 1 (spikes.cu) queues the active rows; stage 2 (here) is a persistent grid
// of warps that walks the queue.  A fixed-number row is split into chunks of
// `chunk` entries so that a few hundred active rows still fill the machine; each
// lane streams indices (and weights) with 128-bit loads and issues one
// red.global.add.f32 per synapse.  HBM traffic per event is 4 B (index) + 4 B
// (heterogeneous weight); the adds resolve in L2.
#include "bsx_tuning.h"
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

// HAS_X: multiply by the float input value (plain sparse vecmat); otherwise every
// queued row is a unit event.
template <bool HETERO, bool HAS_X>
__global__ void __launch_bounds__(256)
scatter_queue_kernel(RowMap rm, const int32_t* __restrict__ idx, const float* __restrict__ w,
                     const int32_t* __restrict__ count_ptr, const uint32_t* __restrict__ entries,
                     const float* __restrict__ x, float* __restrict__ out, int64_t n_pre, int64_t n_post,
                     int64_t batch, int chunks_per_row, int chunk, bool vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t count = *count_ptr;
  // Few active rows: small chunks spread each row over many warps (latency).  Many:
  // eight times larger chunks, fewer and longer streams per warp (throughput).
  if (chunks_per_row > 1 && count * chunks_per_row > 4 * nwarps) {
    chunk *= 8;
    chunks_per_row = (chunks_per_row + 7) >> 3;
  }
  const int64_t items = count * chunks_per_row;
  const float w0 = HETERO ? 1.0f : __ldg(w);
  for (int64_t it = warp; it < items; it += nwarps) {
    const int64_t q = it / chunks_per_row;
    const int c = (int)(it - q * chunks_per_row);
    const uint32_t flat = __ldg(entries + q);
    int64_t b = 0, i = flat;
    if (batch > 1) {
      b = flat / n_pre;
      i = flat - b * n_pre;
    }
    int64_t s, e;
    rm.range(i, s, e);
    if (chunks_per_row > 1) {
      s += (int64_t)c * chunk;
      if (s + chunk < e) e = s + chunk;
    }
    float v = HAS_X ? __ldg(x + flat) : 1.0f;
    if (!HETERO) v = __fmul_rn(v, w0);
    scatter_span<HETERO>(idx, w, s, e, lane, v, out + b * n_post, vec_ok);
  }
}

static int launch_scatter(const bsx_conn_t* conn, const int32_t* count_ptr, const uint32_t* entries,
                          const float* x, float* out, int64_t batch, int64_t max_rows, int chunk,
                          int blocks_per_sm, cudaStream_t st) {
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  if (chunk <= 0) chunk = 128;
  if (blocks_per_sm <= 0) blocks_per_sm = 8;
  int cpr = 1;
  if (!conn->indptr && conn->conn_num > chunk) {
    int64_t c = (conn->conn_num + chunk - 1) / chunk;
    if (c > 1 << 20) {  // keep chunks_per_row in int range: widen the chunk instead
      chunk = (int)((conn->conn_num + (1 << 20) - 1) >> 20);
      c = (conn->conn_num + chunk - 1) / chunk;
    }
    cpr = (int)c;
  }
  int64_t blocks = (max_rows * cpr + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)sms * blocks_per_sm) blocks = (int64_t)sms * blocks_per_sm;
  const bool vec_ok = aligned16(conn->indices) && (!conn->hetero || aligned16(conn->weights));
  const RowMap rm = make_rowmap(conn);
  const unsigned g = (unsigned)blocks;
#define BSX_SCATTER(H, X)                                                                            \
  scatter_queue_kernel<H, X><<<g, 256, 0, st>>>(rm, conn->indices, conn->weights, count_ptr, entries, \
                                                x, out, conn->n_pre, conn->n_post, batch, cpr, chunk, vec_ok)
  if (conn->hetero) {
    if (x) BSX_SCATTER(true, true); else BSX_SCATTER(true, false);
  } else {
    if (x) BSX_SCATTER(false, true); else BSX_SCATTER(false, false);
  }
#undef BSX_SCATTER
  BSX_LAUNCH_CHECK("scatter_queue_kernel");
  return BSX_OK;
}

static size_t queue_bytes(int64_t batch, int64_t n_pre) {
  size_t b = sizeof(QueueHeader) + sizeof(uint32_t) * (size_t)batch * (size_t)n_pre;
  return (b + 255) & ~size_t(255);
}

int vecmat_common(const bsx_conn_t* conn, const void* in, int format, const float* x, int64_t batch,
                         float* out, int accumulate, void* ws, size_t ws_bytes, int chunk,
                         int blocks_per_sm, cudaStream_t st) {
  int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (batch == 0 || conn->n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  const int64_t out_n = batch * conn->n_post;
  const bool empty = conn->n_pre == 0 || (!conn->indptr && conn->conn_num == 0);
  if (empty) return accumulate ? BSX_OK : launch_zero(out, out_n, st);
  if (!in) return fail(BSX_ERR_INVALID_ARG, "input vector is NULL");
  if ((double)batch * (double)conn->n_pre >= 4294967296.0)
    return fail(BSX_ERR_UNSUPPORTED, "batch * n_pre must be below 2^32");

  // The variant that keeps output slices in shared memory runs one block per (batch row,
  // slice): it needs about as many of those as there are SMs, and re-reads every active row
  // once per slice.  blocks_per_sm < 0 asks for it wherever it applies; with every tuning
  // argument at 0 it is chosen when the batch fills the GPU and the output has at most two
  // slices (measured at 65 536 columns: 1.0-1.1x the global-atomic kernel at 0.1 % firing,
  // 1.5-2.2x at 1 %, 1.8-2.3x at 10 %, for 64 to 296 vectors).  A positive blocks_per_sm or
  // chunk keeps the global-atomic kernel.
  if (blocks_per_sm < 0 || (blocks_per_sm == 0 && chunk == 0 && scatter_smem_preferred(conn, format, batch))) {
    if (scatter_smem_applies(conn, format, batch))
      return launch_scatter_smem(conn, in, format, x, batch, out, accumulate, st);
    blocks_per_sm = 0;
  }
  // A few spike vectors (the per-step call of a simulation): a memset node and ONE kernel that
  // lists the active rows in shared memory and scatters them; the workspace stays untouched
  // (it is still checked, so that a caller's sizing error shows at any input size).  Explicit
  // tuning arguments keep the queue + scatter launches.
  if (blocks_per_sm == 0 && chunk == 0 && scatter_fused_applies(conn, in, format, batch)) {
    if (format != BSX_SPK_LIST) {
      if (!ws || (reinterpret_cast<uintptr_t>(ws) & 15)) return fail(BSX_ERR_WORKSPACE, "workspace NULL or not 16-byte aligned");
      if (ws_bytes < queue_bytes(batch, conn->n_pre))
        return fail(BSX_ERR_WORKSPACE, "workspace too small: %zu < %zu", ws_bytes, queue_bytes(batch, conn->n_pre));
    }
    return launch_scatter_fused(conn, in, format, x, batch, out, accumulate, st);
  }
  if (format == BSX_SPK_LIST) {
    if (batch != 1) return fail(BSX_ERR_UNSUPPORTED, "an index list describes one spike vector (batch 1)");
    if (!accumulate) {
      rc = launch_zero(out, out_n, st);
      if (rc) return rc;
    }
    const int32_t* list = static_cast<const int32_t*>(in);
    return launch_scatter(conn, list, reinterpret_cast<const uint32_t*>(list + 1), nullptr, out, 1,
                          conn->n_pre, chunk, blocks_per_sm, st);
  }
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 15)) return fail(BSX_ERR_WORKSPACE, "workspace NULL or not 16-byte aligned");
  if (ws_bytes < queue_bytes(batch, conn->n_pre))
    return fail(BSX_ERR_WORKSPACE, "workspace too small: %zu < %zu", ws_bytes, queue_bytes(batch, conn->n_pre));
  QueueHeader* hdr = static_cast<QueueHeader*>(ws);
  uint32_t* entries = reinterpret_cast<uint32_t*>(hdr + 1);
  rc = launch_compact(in, format, batch, conn->n_pre, hdr, entries, accumulate ? nullptr : out,
                      accumulate ? 0 : out_n, st);
  if (rc) return rc;
  return launch_scatter(conn, &hdr->count, entries, x, out, batch, batch * conn->n_pre, chunk,
                        blocks_per_sm, st);
}

}  // namespace bsx

using namespace bsx;

extern "C" {

size_t bsx_event_vecmat_workspace_bytes(int64_t batch, int64_t n_pre) {
  if (batch < 0 || n_pre < 0) return 0;
  return queue_bytes(batch, n_pre);
}

int bsx_event_vecmat_tuned(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                           float* out, int accumulate, void* workspace, size_t workspace_bytes,
                           int chunk, int blocks_per_sm, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_tuned");
  if (spike_format < BSX_SPK_BOOL8 || spike_format > BSX_SPK_LIST)
    return fail(BSX_ERR_INVALID_ARG, "unknown spike format %d", spike_format);
  return vecmat_common(conn, spikes, spike_format, nullptr, batch, out, accumulate, workspace,
                       workspace_bytes, chunk, blocks_per_sm, as_stream(stream));
}

int bsx_event_vecmat_variant(const bsx_conn_t* conn, int spike_format, int64_t batch) {
  if (spike_format < BSX_SPK_BOOL8 || spike_format > BSX_SPK_LIST)
    return fail(BSX_ERR_INVALID_ARG, "unknown spike format %d", spike_format);
  const int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  return scatter_smem_preferred(conn, spike_format, batch) ? BSX_VECMAT_SHARED_SLICES : BSX_VECMAT_GLOBAL_ATOMICS;
}

int bsx_event_vecmat_chained(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                             float* out, float* next_out, bsx_stream_t stream) {
  BSX_TRACE("bsx_event_vecmat_chained");
  const int rc = check_conn(conn);
  if (rc) return rc;
  if (batch < 0) return fail(BSX_ERR_INVALID_ARG, "negative batch");
  if (spike_format != BSX_SPK_BOOL8 && spike_format != BSX_SPK_F32 && spike_format != BSX_SPK_BITS32 &&
      spike_format != BSX_SPK_LIST)
    return fail(BSX_ERR_INVALID_ARG, "unknown spike format");
  if (batch == 0 || conn->n_post == 0) return BSX_OK;
  if (!out) return fail(BSX_ERR_INVALID_ARG, "out is NULL");
  if (next_out == out) return fail(BSX_ERR_INVALID_ARG, "next_out must be another buffer than out");
  cudaStream_t st = as_stream(stream);
  const bool empty = conn->n_pre == 0 || (!conn->indptr && conn->conn_num == 0);
  if (empty) return next_out ? launch_zero(next_out, batch * conn->n_post, st) : BSX_OK;
  if (!spikes) return fail(BSX_ERR_INVALID_ARG, "input vector is NULL");
  if (!scatter_fused_applies(conn, spikes, spike_format, batch))
    return fail(BSX_ERR_UNSUPPORTED, "the chained call takes up to 128 KB of 16-byte aligned spike input");
  return launch_scatter_fused(conn, spikes, spike_format, nullptr, batch, out, /*accumulate=*/1, st, next_out);
}

int bsx_event_vecmat_launches(const bsx_conn_t* conn, int spike_format, int64_t batch) {
  const int v = bsx_event_vecmat_variant(conn, spike_format, batch);
  if (v < 0) return v;
  if (v == BSX_VECMAT_SHARED_SLICES) return 1;
  if (scatter_fused_fits(conn, spike_format, batch)) return 1;   // given 16-byte aligned buffers
  return 2;                                                      // (clear | compaction + clear) and scatter
}

int bsx_event_vecmat(const bsx_conn_t* conn, const void* spikes, int spike_format, int64_t batch,
                     float* out, int accumulate, void* workspace, size_t workspace_bytes,
                     bsx_stream_t stream) {
  return bsx_event_vecmat_tuned(conn, spikes, spike_format, batch, out, accumulate, workspace,
                                workspace_bytes, 0, 0, stream);
}

int bsx_float_vecmat(const bsx_conn_t* conn, const float* x, int64_t batch, float* out, int accumulate,
                     void* workspace, size_t workspace_bytes, bsx_stream_t stream) {
  BSX_TRACE("bsx_float_vecmat");
  return vecmat_common(conn, x, BSX_SPK_F32, x, batch, out, accumulate, workspace, workspace_bytes, 0, 0,
                       as_stream(stream));
}

}  // extern "C"
