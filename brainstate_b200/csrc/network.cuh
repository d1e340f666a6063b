// Device code shared by the network step kernels: projection descriptor, background
// drive hash, the exponential factor and the arithmetic of one neuron for one step.
#pragma once

#include "common.cuh"

namespace bsx {

struct ProjDev {
  RowMap rm;
  const int32_t* idx;
  const float* w;
  int hetero;
  int cpr;      // chunks per row
  bool vec_ok;
};

// Counter-based background drive: neuron `gid` receives one external excitatory
// event at step `step` when a 32-bit hash of (seed, gid, step) falls below the
// threshold.  Integer arithmetic only, so a host restatement matches bit for bit.
__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__host__ __device__ __forceinline__ uint32_t drive_hash(uint32_t seed, uint32_t gid, uint32_t step) {
  return mix32(mix32(gid + seed * 0x9e3779b9u) ^ (step * 0x85ebca6bu + 0xc2b2ae35u));
}

// (exp(z) - 1) / z.  For |z| <= 0.125 (every realistic dt * df/dV) the degree-5 Taylor
// polynomial 1 + z/2 + ... + z^5/720 in Horner form, each multiply and add rounded
// separately in float32 so that a host restatement doing the same operations matches
// bit for bit.  The first dropped term, z^6/5040, is below 8e-10 there and the result
// stays within one float32 ulp of the float64 value (0.57 ulp at worst); otherwise
// evaluated in double and rounded once.
__device__ __forceinline__ float exprel_once(float z) {
  if (fabsf(z) <= 0.125f) {
    float p = 0.0013888889f;                                  // 1/720
    p = __fadd_rn(__fmul_rn(p, z), 0.008333334f);             // 1/120
    p = __fadd_rn(__fmul_rn(p, z), 0.041666668f);             // 1/24
    p = __fadd_rn(__fmul_rn(p, z), 0.16666667f);              // 1/6
    p = __fadd_rn(__fmul_rn(p, z), 0.5f);
    p = __fadd_rn(__fmul_rn(p, z), 1.0f);
    return p;
  }
  const double zd = (double)z;
  return (float)(expm1(zd) / zd);
}

// The arithmetic of one neuron for one step: synapse decay + increment (+ background
// drive), membrane update, threshold, reset, refractory count.  Pure: state in, state out.
struct NeuronOut {
  float ge, gi, V;
  int32_t r;
  bool spk;
};

// MODEL 0 reads the synapse model and the background drive from the parameters; the others fix them
// at compile time (1: conductance-based, no drive; 2: current-based, no drive; 3: current-based with
// drive), which takes the uniform branches (and, without drive, the hash) out of the loop of a kernel
// that is bound by instruction issue.
template <int MODEL>
__device__ __forceinline__ NeuronOut neuron_math_m(const bsx_lif_params_t& p, float de, float di, float ge0,
                                                   float gi0, float V, int32_t r, uint32_t gid, int64_t step) {
  const bool coba = MODEL == 0 ? (p.coba != 0) : MODEL == 1;
  if ((MODEL == 3 || (MODEL == 0 && p.ext_threshold)) && drive_hash(p.ext_seed, gid, (uint32_t)step) < p.ext_threshold)
    de = __fadd_rn(de, p.ext_weight);
  NeuronOut o;
  o.ge = __fadd_rn(__fmul_rn(ge0, p.decay_e), de);
  o.gi = __fadd_rn(__fmul_rn(gi0, p.decay_i), di);
  float cur;
  if (coba) cur = __fadd_rn(__fmul_rn(o.ge, __fsub_rn(p.E_e, V)), __fmul_rn(o.gi, __fsub_rn(p.E_i, V)));
  else cur = __fadd_rn(o.ge, o.gi);
  const float drive = __fmul_rn(p.R, __fadd_rn(cur, p.I_ext));
  const float num = __fadd_rn(__fsub_rn(p.V_rest, V), drive);
  float Vn;
  if (coba) {
    const float f = __fmul_rn(num, p.inv_tau_m);
    const float gsum = __fadd_rn(o.ge, o.gi);
    const float J = __fmul_rn(-__fadd_rn(1.0f, __fmul_rn(p.R, gsum)), p.inv_tau_m);
    const float gain = __fmul_rn(p.dt, exprel_once(__fmul_rn(p.dt, J)));
    Vn = __fadd_rn(V, __fmul_rn(gain, f));
  } else {
    Vn = __fadd_rn(V, __fmul_rn(p.cuba_gain, num));
  }
  const bool refractory = r > 0;
  if (refractory) Vn = V;
  o.spk = (Vn >= p.V_th) && !refractory;
  o.V = o.spk ? p.V_reset : Vn;
  o.r = o.spk ? p.ref_steps : (r > 0 ? r - 1 : 0);
  return o;
}

__device__ __forceinline__ NeuronOut neuron_math(const bsx_lif_params_t& p, float de, float di, float ge0,
                                                 float gi0, float V, int32_t r, uint32_t gid, int64_t step) {
  return neuron_math_m<0>(p, de, di, ge0, gi0, V, r, gid, step);
}

inline int make_proj(const bsx_conn_t* c, int chunk, ProjDev* out) {
  int rc = check_conn(c);
  if (rc) return rc;
  out->rm = make_rowmap(c);
  out->idx = c->indices;
  out->w = c->weights;
  out->hetero = c->hetero;
  out->vec_ok = aligned16(c->indices) && (!c->hetero || aligned16(c->weights));
  out->cpr = 1;
  if (!c->indptr && c->conn_num > chunk) out->cpr = (int)((c->conn_num + chunk - 1) / chunk);
  return BSX_OK;
}

}  // namespace bsx
