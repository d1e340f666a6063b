// Diagnostics, small utilities and the host-side connectivity generator.
#include <new>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace bsx {

static thread_local char g_error[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_error, sizeof(g_error), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return BSX_ERR_CUDA;
}

int check_conn(const bsx_conn_t* c) {
  if (!c) return fail(BSX_ERR_INVALID_ARG, "conn is NULL");
  if (c->n_pre < 0 || c->n_post < 0) return fail(BSX_ERR_INVALID_ARG, "negative matrix size");
  if (c->n_post > INT32_MAX || c->n_pre > INT32_MAX)
    return fail(BSX_ERR_UNSUPPORTED, "n_pre and n_post must fit int32 indices");
  if (!c->indptr && c->conn_num < 0) return fail(BSX_ERR_INVALID_ARG, "negative conn_num");
  bool empty = c->n_pre == 0 || (!c->indptr && c->conn_num == 0);
  if (!empty && !c->indices) return fail(BSX_ERR_INVALID_ARG, "indices is NULL");
  if (!c->weights) return fail(BSX_ERR_INVALID_ARG, "weights is NULL");
  if (c->nnz < 0 || (!c->indptr && c->nnz != c->n_pre * c->conn_num))
    return fail(BSX_ERR_INVALID_ARG, "nnz does not match the layout");
  return BSX_OK;
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

__global__ void fill_kernel(float* __restrict__ dst, int64_t n, float v) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = v;
}

// ---- MT19937 as NumPy's legacy RandomState drives it ------------------------
struct Mt19937 {
  static const int N = 624, M = 397;
  uint32_t key[N];
  int pos;
  explicit Mt19937(uint32_t seed) {
    key[0] = seed;
    for (int i = 1; i < N; ++i) key[i] = 1812433253u * (key[i - 1] ^ (key[i - 1] >> 30)) + (uint32_t)i;
    pos = N;
  }
  static inline uint32_t twist(uint32_t hi, uint32_t lo, uint32_t far) {
    uint32_t y = (hi & 0x80000000u) | (lo & 0x7fffffffu);
    return far ^ (y >> 1) ^ (-(int32_t)(y & 1u) & 0x9908b0dfu);
  }
  void refill() {
    int i = 0;
    for (; i < N - M; ++i) key[i] = twist(key[i], key[i + 1], key[i + M]);
    for (; i < N - 1; ++i) key[i] = twist(key[i], key[i + 1], key[i + M - N]);
    key[N - 1] = twist(key[N - 1], key[0], key[M - 1]);
    pos = 0;
  }
  inline uint32_t next() {
    if (pos == N) refill();
    uint32_t y = key[pos++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
  }
};

}  // namespace bsx

using namespace bsx;

extern "C" {

int bsx_version(void) { return BSX_VERSION; }

const char* bsx_last_error_string(void) { return g_error; }

const char* bsx_status_name(int status) {
  switch (status) {
    case BSX_OK: return "BSX_OK";
    case BSX_ERR_INVALID_ARG: return "BSX_ERR_INVALID_ARG";
    case BSX_ERR_CUDA: return "BSX_ERR_CUDA";
    case BSX_ERR_INDEX_RANGE: return "BSX_ERR_INDEX_RANGE";
    case BSX_ERR_WORKSPACE: return "BSX_ERR_WORKSPACE";
    case BSX_ERR_UNSUPPORTED: return "BSX_ERR_UNSUPPORTED";
    case BSX_ERR_TIMEOUT: return "BSX_ERR_TIMEOUT";
    case BSX_ERR_NONFINITE: return "BSX_ERR_NONFINITE";
    default: return "BSX_ERR_UNKNOWN";
  }
}

int bsx_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int bsx_read_status(const int32_t* status_word, int32_t* host_status, bsx_stream_t stream) {
  if (!status_word || !host_status) return fail(BSX_ERR_INVALID_ARG, "status pointers must not be NULL");
  BSX_CUDA(cudaMemcpyAsync(host_status, status_word, sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
  BSX_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return BSX_OK;
}

int bsx_fill_f32(float* dst, int64_t n, float value, bsx_stream_t stream) {
  if (n < 0 || (!dst && n > 0)) return fail(BSX_ERR_INVALID_ARG, "bsx_fill_f32: bad destination");
  if (n == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (n + 255) / 256;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  fill_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(dst, n, value);
  BSX_LAUNCH_CHECK("fill_kernel");
  return BSX_OK;
}

int64_t bsx_host_fixed_num_indices(uint32_t seed, int64_t n_pre, int64_t n_post, int64_t conn_num,
                                   int64_t row_begin, int64_t row_end, int64_t col_begin,
                                   int64_t col_end, int32_t* host_out, int32_t* host_row_counts) {
  if (n_pre < 0 || n_post < 1 || conn_num < 0 || n_post > (int64_t)INT32_MAX)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_fixed_num_indices: bad sizes");
  if (row_begin < 0 || row_end > n_pre || row_begin > row_end)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_fixed_num_indices: bad row range");
  const bool filter = col_begin < col_end;
  if (filter && (col_begin < 0 || col_end > n_post))
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_fixed_num_indices: bad column range");
  if (filter && !host_row_counts)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_fixed_num_indices: row counts required with a column range");
  if (!host_out && row_end > row_begin && conn_num > 0)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_fixed_num_indices: output is NULL");

  const uint32_t top = (uint32_t)(n_post - 1);
  int64_t written = 0;
  if (top == 0) {  // a one-value range consumes no draws
    for (int64_t r = row_begin; r < row_end; ++r) {
      int32_t kept = 0;
      for (int64_t k = 0; k < conn_num; ++k)
        if (!filter || col_begin == 0) { host_out[written++] = 0; ++kept; }
      if (host_row_counts) host_row_counts[r - row_begin] = kept;
    }
    return written;
  }
  uint32_t mask = top;
  mask |= mask >> 1; mask |= mask >> 2; mask |= mask >> 4; mask |= mask >> 8; mask |= mask >> 16;
  Mt19937 mt(seed);
  // rows before the requested range: replay the stream, keep nothing
  for (int64_t n = row_begin * conn_num; n > 0; --n) {
    uint32_t v;
    do { v = mt.next() & mask; } while (v > top);
  }
  const uint32_t c0 = (uint32_t)(filter ? col_begin : 0), c1 = (uint32_t)(filter ? col_end : n_post);
  for (int64_t r = row_begin; r < row_end; ++r) {
    int32_t kept = 0;
    for (int64_t k = 0; k < conn_num; ++k) {
      uint32_t v;
      do { v = mt.next() & mask; } while (v > top);
      if (v >= c0 && v < c1) { host_out[written++] = (int32_t)(v - c0); ++kept; }
    }
    if (host_row_counts) host_row_counts[r - row_begin] = kept;
  }
  return written;
}

// ---- stateful form of the generator: one stream, drawn in row chunks -----------
void* bsx_host_gen_new(uint32_t seed) { return new (std::nothrow) Mt19937(seed); }

void bsx_host_gen_free(void* gen) { delete static_cast<Mt19937*>(gen); }

int64_t bsx_host_gen_rows(void* gen, int64_t rows, int64_t n_post, int64_t conn_num, int64_t col_begin,
                          int64_t col_end, int32_t* host_out, int16_t* host_k_out, int32_t* host_row_counts) {
  if (!gen) return fail(BSX_ERR_INVALID_ARG, "bsx_host_gen_rows: generator is NULL");
  if (rows < 0 || n_post < 1 || conn_num < 0 || n_post > (int64_t)INT32_MAX || conn_num > 32767)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_gen_rows: bad sizes (conn_num must be below 32768)");
  const bool filter = col_begin < col_end;
  if (filter && (col_begin < 0 || col_end > n_post))
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_gen_rows: bad column range");
  if (!host_out && rows > 0 && conn_num > 0) return fail(BSX_ERR_INVALID_ARG, "bsx_host_gen_rows: output is NULL");
  Mt19937& mt = *static_cast<Mt19937*>(gen);
  const uint32_t top = (uint32_t)(n_post - 1);
  uint32_t mask = top;
  mask |= mask >> 1; mask |= mask >> 2; mask |= mask >> 4; mask |= mask >> 8; mask |= mask >> 16;
  const uint32_t c0 = (uint32_t)(filter ? col_begin : 0), c1 = (uint32_t)(filter ? col_end : n_post);
  int64_t written = 0;
  for (int64_t r = 0; r < rows; ++r) {
    int32_t kept = 0;
    for (int64_t k = 0; k < conn_num; ++k) {
      uint32_t v = 0;
      if (top) {  // a one-value range consumes no draws
        do { v = mt.next() & mask; } while (v > top);
      }
      if (v >= c0 && v < c1) {
        host_out[written] = (int32_t)(v - c0);
        if (host_k_out) host_k_out[written] = (int16_t)k;
        ++written;
        ++kept;
      }
    }
    if (host_row_counts) host_row_counts[r] = kept;
  }
  return written;
}

// Rows of conn_num DISTINCT targets each (sampling without replacement), from the same
// generator: bounded draws in stream order, a draw that repeats a target of the current
// row is dropped.  Every ordered conn_num-subset is equally likely.  This is the
// library's sampler for `allow_multi_conn=False`
// (brainstate/nn/_event_fixedprob.py:39-62); it does not reproduce the reference's
// numbers, which come from JAX's threefry generator.
int64_t bsx_host_distinct_indices(uint32_t seed, int64_t n_pre, int64_t n_post, int64_t conn_num,
                                  int32_t* host_out) {
  if (n_pre < 0 || n_post < 1 || conn_num < 0 || n_post > (int64_t)INT32_MAX)
    return fail(BSX_ERR_INVALID_ARG, "bsx_host_distinct_indices: bad sizes");
  if (conn_num > n_post) return fail(BSX_ERR_INVALID_ARG, "cannot draw %lld distinct targets out of %lld",
                                     (long long)conn_num, (long long)n_post);
  if (!host_out && n_pre * conn_num > 0) return fail(BSX_ERR_INVALID_ARG, "bsx_host_distinct_indices: output is NULL");
  const uint32_t top = (uint32_t)(n_post - 1);
  uint32_t mask = top;
  mask |= mask >> 1; mask |= mask >> 2; mask |= mask >> 4; mask |= mask >> 8; mask |= mask >> 16;
  const size_t words = (size_t)((n_post + 63) / 64);
  uint64_t* seen = new (std::nothrow) uint64_t[words]();
  if (!seen) return fail(BSX_ERR_INVALID_ARG, "bsx_host_distinct_indices: out of host memory");
  Mt19937 mt(seed);
  for (int64_t r = 0; r < n_pre; ++r) {
    int32_t* row = host_out + r * conn_num;
    for (int64_t k = 0; k < conn_num;) {
      uint32_t v = 0;
      if (top) {
        do { v = mt.next() & mask; } while (v > top);
      }
      uint64_t& w = seen[v >> 6];
      const uint64_t bit = 1ull << (v & 63);
      if (w & bit) continue;
      w |= bit;
      row[k++] = (int32_t)v;
    }
    for (int64_t k = 0; k < conn_num; ++k) seen[(uint32_t)row[k] >> 6] = 0;   // clear only what was set
  }
  delete[] seen;
  return n_pre * conn_num;
}

}  // extern "C"
