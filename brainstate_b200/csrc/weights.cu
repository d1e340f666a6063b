// Position-keyed synaptic weights: w(row, k) = sign * exp(mu + sigma * z(row, k)) with
// z a standard normal derived from a 32-bit hash of (seed, global row, k).  Because the
// value depends only on the position of the synapse in the full matrix, every rank of a
// sharded network can fill the weights of the synapses it kept without seeing the rest,
// and a host restatement reproduces them (integer hash; the transcendental part is
// evaluated in double and rounded once).
#include "common.cuh"
#include "internal.cuh"

namespace bsx {

__host__ __device__ __forceinline__ uint32_t wmix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

__host__ __device__ __forceinline__ float lognormal_at(uint32_t seed, uint32_t row, uint32_t k, double mu,
                                                       double sigma, float sign) {
  const uint32_t h = wmix32(wmix32(row + seed * 0x9e3779b9u) ^ (k * 0x85ebca6bu + 0x27d4eb2fu));
  const uint32_t g = wmix32(h ^ 0x165667b1u);
  const double u1 = ((double)h + 1.0) * (1.0 / 4294967296.0);   // (0, 1]
  const double u2 = (double)g * (1.0 / 4294967296.0);           // [0, 1)
  const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
  return sign * (float)exp(mu + sigma * z);
}

__global__ void __launch_bounds__(256)
lognormal_kernel(RowMap rm, const int16_t* __restrict__ kpos, int64_t n_rows, int64_t row0, uint32_t seed,
                 double mu, double sigma, float sign, float* __restrict__ w) {
  const int lane = threadIdx.x & 31;
  const int64_t wstep = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n_rows; row += wstep) {
    int64_t s, e;
    rm.range(row, s, e);
    for (int64_t p = s + lane; p < e; p += 32) {
      const uint32_t k = kpos ? (uint32_t)(uint16_t)kpos[p] : (uint32_t)(p - s);
      w[p] = lognormal_at(seed, (uint32_t)(row0 + row), k, mu, sigma, sign);
    }
  }
}

}  // namespace bsx

using namespace bsx;

extern "C" {

int bsx_lognormal_weights(const bsx_conn_t* conn, const int16_t* kpos, int64_t row0, uint32_t seed, double mu,
                          double sigma, float sign, float* weights_out, bsx_stream_t stream) {
  if (!conn || !weights_out) return fail(BSX_ERR_INVALID_ARG, "bsx_lognormal_weights: NULL argument");
  if (conn->n_pre < 0 || (!conn->indptr && conn->conn_num < 0)) return fail(BSX_ERR_INVALID_ARG, "bad layout");
  if (conn->n_pre == 0 || conn->nnz == 0) return BSX_OK;
  int sms = sm_count();
  if (sms <= 0) return fail(BSX_ERR_CUDA, "no CUDA device");
  int64_t blocks = (conn->n_pre + 7) / 8;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  lognormal_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(make_rowmap(conn), kpos, conn->n_pre, row0,
                                                                    seed, mu, sigma, sign, weights_out);
  BSX_LAUNCH_CHECK("lognormal_kernel");
  return BSX_OK;
}

float bsx_lognormal_weight_at(uint32_t seed, uint32_t row, uint32_t k, double mu, double sigma, float sign) {
  return lognormal_at(seed, row, k, mu, sigma, sign);
}

}  // extern "C"
