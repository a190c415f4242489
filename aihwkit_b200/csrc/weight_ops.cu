// Weight operations between updates: decay, diffusion, clipping, column reset, uniform
// re-initialisation. Per-element device rules of PulsedRPUDevice
// (src/rpucuda/rpu_pulsed_device.cpp:362-490); for the floating-point (ideal) device the rules of
// RPUSimple / SimpleRPUDevice (src/rpucuda/rpu.cpp:1556-1625, rpu_simple_device.cpp:149-169) and
// WeightClipper::apply (src/rpucuda/weight_clipper.cpp:38-118).
//
// All kernels are one pass over the weights [x_size][d_size] (plus the 16-byte bounds and the
// 16-byte decay / diffusion / reset record per element): HBM-bound, 24-40 B per weight.
#include "tile.h"

#include <algorithm>
#include <cmath>
#include <vector>

namespace ab200 {

enum : uint32_t {
  TAG_DIFFUSE = 0x70000000u,
  TAG_RESET = 0x71000000u,
  TAG_UNIFORM_INIT = 0x72000000u,
  TAG_DRIFT = 0x73000000u,
  TAG_MODIFY = 0x74000000u,
};

namespace {

// par4 = {scale_up, scale_down, max_bound, min_bound}, par3 = {decay_scale, diffusion, reset_bias, -}
__global__ void __launch_bounds__(256)
    decayKernel(float *w, const float4 *par4, const float4 *par3, long long n, long long first_bias,
                float alpha, int use_alpha) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= n) {
    return;
  }
  const float4 q = par4[t], r = par3[t];
  // w = (w - b) * s + b with s = decay_scale, or 1 + alpha * (decay_scale - 1)
  float s = use_alpha ? __fadd_rn(1.0f, __fmul_rn(alpha, __fsub_rn(r.x, 1.0f))) : r.x;
  if (t >= first_bias) {
    s = 1.0f; // bias column does not decay
  }
  float v = __fadd_rn(__fmul_rn(__fsub_rn(w[t], r.z), s), r.z);
  v = fminf(v, q.z);
  v = fmaxf(v, q.w);
  w[t] = v;
}

// Largest |w| over the first n elements (float bits compare like unsigned integers for w >= 0).
__global__ void __launch_bounds__(256) absMaxKernel(const float *w, long long n, unsigned int *out) {
  float a = 0.0f;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n;
       t += (long long)gridDim.x * blockDim.x) {
    a = fmaxf(a, fabsf(w[t]));
  }
  for (int o = 16; o > 0; o >>= 1) {
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  }
  if ((threadIdx.x & 31) == 0 && a > 0.0f) {
    atomicMax(out, __float_as_uint(a));
  }
}

// WeightModifier::apply (src/rpucuda/weight_modifier.cpp:31-215) for one element: fb = f(w).
// Elements t >= n_mod (the last input column when copy_last_column is set) are copied.
// `amax_dev`: largest |w| of the modified elements, or null for the assumed value in g.amax.
struct ModifyArgs {
  int type, sto_round, n_coeffs;
  float std_dev, res, dorefa_clip, pdrop, amax, g_max;
  float coeffs[AB200_WMOD_MAX_COEFFS];
};
__device__ __forceinline__ float modRound(float v, float res, bool sto, float u) {
  // getDiscretizedValueRound (src/rpucuda/utility_functions.h:195-203)
  if (!(res > 0.0f)) {
    return v;
  }
  // roundf here: halves away from zero, unlike the DAC / ADC steps
  return sto ? __fmul_rn(roundf(__fadd_rn(__fdiv_rn(v, res), __fadd_rn(u, -0.5f))), res)
             : __fmul_rn(roundf(__fdiv_rn(v, res)), res);
}
__global__ void __launch_bounds__(256)
    modifyKernel(const float *w, float *fb, long long n, long long n_mod, const unsigned int *amax_dev,
                 ModifyArgs g, PhiloxKey key, uint32_t call) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= n) {
    return;
  }
  float v = w[t];
  if (t >= n_mod) {
    fb[t] = v;
    return;
  }
  float amax = g.amax;
  if (amax_dev) {
    amax = __uint_as_float(*amax_dev);
    amax = amax > 0.0f ? amax : 1.0f;
  }
  uint32_t r[4];
  philox4x32<7>((uint32_t)t, (uint32_t)(t >> 32), call, TAG_MODIFY, key, r);
  float z, z_unused;
  boxMuller16(r[1], z, z_unused);
  const float u = u01(r[0]);
  const bool sto = g.sto_round != 0;
  switch (g.type) {
  case AB200_WMOD_DISCRETIZE:
    if (g.res > 0.0f) {
      v = __fmul_rn(amax, modRound(__fdiv_rn(v, amax), g.res, sto, u));
    }
    break;
  case AB200_WMOD_MULT_NORMAL:
    if (g.std_dev > 0.0f) {
      v = __fadd_rn(v, __fmul_rn(__fmul_rn(v, __fmul_rn(g.std_dev, amax)), z));
    }
    break;
  case AB200_WMOD_ADD_NORMAL:
    if (g.std_dev > 0.0f) {
      v = __fadd_rn(v, __fmul_rn(__fmul_rn(g.std_dev, amax), z));
    }
    break;
  case AB200_WMOD_DISCRETIZE_ADD_NORMAL: {
    const float std = __fmul_rn(g.std_dev, amax);
    if (g.res > 0.0f || std > 0.0f) {
      v = __fmul_rn(amax, modRound(__fdiv_rn(v, amax), g.res, sto, u));
      v = __fadd_rn(v, __fmul_rn(std, z));
    }
    break;
  }
  case AB200_WMOD_DOREFA:
    if (g.res > 0.0f) {
      const float scale = fabsf(__fdiv_rn(g.dorefa_clip, tanhf(amax)));
      v = modRound(__fmul_rn(tanhf(v), scale), g.res, sto, u);
    }
    break;
  case AB200_WMOD_POLY:
  case AB200_WMOD_PROG_NOISE:
    if (g.std_dev > 0.0f && g.n_coeffs > 0) {
      const float aw = __fdiv_rn(fabsf(v), amax);
      float paw = 1.0f, sig = g.coeffs[0];
      for (int j = 1; j < g.n_coeffs; j++) {
        paw = __fmul_rn(paw, aw);
        sig = __fadd_rn(sig, __fmul_rn(g.coeffs[j], paw));
      }
      const float std = g.type == AB200_WMOD_POLY ? g.std_dev : __fdiv_rn(g.std_dev, g.g_max);
      sig = __fmul_rn(sig, std);
      const float nv = __fadd_rn(v, __fmul_rn(__fmul_rn(amax, sig), z));
      v = g.type == AB200_WMOD_POLY ? nv : (v < 0.0f ? -fabsf(nv) : fabsf(nv));
    }
    break;
  default: // Copy, DropConnect
    break;
  }
  if (g.pdrop > 0.0f && u01(r[2]) < g.pdrop) {
    v = 0.0f;
  }
  fb[t] = v;
}

// WeightDrifter::apply (src/rpucuda/weight_drifter.cpp:111-157) for one element, followed by
// WeightDrifter::saturate (:101-108) when the device has bounds. `nu_el` null: one exponent for
// all elements (simple drift).
struct DriftArgs {
  float nu, nu_std, wg_ratio, g_offset, w_offset, nu_k, log_g0, reset_tol, w_read_std, a;
};
__global__ void __launch_bounds__(256)
    driftKernel(float *w, float *prev, float *w0, float *t_set, const float *nu_el,
                const float4 *par4, long long n, float now, DriftArgs g, PhiloxKey key,
                uint32_t call) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= n) {
    return;
  }
  float z[4] = {0.f, 0.f, 0.f, 0.f};
  if (g.nu_std > 0.0f || g.w_read_std > 0.0f) {
    float zz[4];
    gauss4(key, (uint64_t)(t >> 1), call, TAG_DRIFT, zz);
    z[0] = zz[(t & 1) * 2];
    z[1] = zz[(t & 1) * 2 + 1];
  }
  float v = w[t];
  if (fabsf(__fsub_rn(prev[t], v)) > g.reset_tol) {
    // written since the last call: the drift starts again from here
    t_set[t] = now;
    w0[t] = v;
  } else {
    float nu = nu_el ? nu_el[t] : g.nu;
    if (g.nu_std > 0.0f) {
      nu = __fadd_rn(nu, __fmul_rn(__fmul_rn(g.nu_std, nu), z[0]));
    }
    if (g.nu_k != 0.0f) {
      nu = __fadd_rn(__fsub_rn(nu, __fmul_rn(g.nu_k, logf(__fadd_rn(__fdiv_rn(__fsub_rn(v, g.w_offset),
                                                                         g.wg_ratio),
                                                               g.g_offset)))),
                     __fmul_rn(g.nu_k, g.log_g0));
    }
    const float dt = fmaxf(__fsub_rn(now, t_set[t]), 1.0f);
    const float sc = powf(dt, -nu);
    v = __fmul_rn(w0[t], sc);
    if (g.a != 0.0f) {
      v = __fadd_rn(v, __fmul_rn(g.a, __fsub_rn(sc, 1.0f)));
    }
  }
  if (g.w_read_std > 0.0f) {
    v = __fadd_rn(v, __fmul_rn(g.w_read_std, z[1]));
  }
  float pv = v;
  if (par4) {
    const float4 q = par4[t];
    v = fminf(fmaxf(q.w, v), q.z);
    pv = v;
  }
  prev[t] = pv;
  w[t] = v;
}

__global__ void __launch_bounds__(256)
    scaleKernel(float *w, long long n, long long first_bias, float scale) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n && t < first_bias) {
    w[t] = __fmul_rn(w[t], scale);
  }
}

// w += rate * N(0,1), then the element's bounds (par4 null: floating-point tile, one rate, no bounds)
__global__ void __launch_bounds__(256)
    diffuseKernel(float *w, const float4 *par4, const float4 *par3, long long n, float rate,
                  PhiloxKey key, uint32_t call) {
  const long long t4 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t4 * 4 >= n) {
    return;
  }
  float z[4];
  gauss4(key, (uint64_t)t4, call, TAG_DIFFUSE, z);
  for (int k = 0; k < 4; k++) {
    const long long t = t4 * 4 + k;
    if (t < n) {
      float v = w[t];
      if (par4) {
        const float4 q = par4[t];
        v += par3[t].y * z[k];
        v = fminf(v, q.z);
        v = fmaxf(v, q.w);
      } else {
        v += rate * z[k];
      }
      w[t] = v;
    }
  }
}

// device bounds, optionally tightened to [-clip, clip] (clip < 0: bounds only)
__global__ void __launch_bounds__(256)
    clipBoundsKernel(float *w, const float4 *par4, long long n, float clip) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= n) {
    return;
  }
  float hi = clip, lo = -clip;
  if (par4) {
    const float4 q = par4[t];
    hi = clip < 0.0f ? q.z : fminf(q.z, clip);
    lo = clip < 0.0f ? q.w : fmaxf(q.w, -clip);
  }
  w[t] = fmaxf(fminf(w[t], hi), lo);
}

// sums for the data-dependent clip values: acc[0] = sum w, acc[1] = sum w^2 (double), and
// rowmax[i] = max_j |w_ij| as float bits (non-negative floats order like unsigned integers)
__global__ void __launch_bounds__(256)
    clipStatsKernel(const float *w, long long n, int d_size, double *acc, unsigned int *rowmax) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  double s = 0.0, s2 = 0.0;
  if (t < n) {
    const float v = w[t];
    s = v;
    s2 = (double)v * v;
    if (rowmax) {
      atomicMax(&rowmax[t % d_size], __float_as_uint(fabsf(v)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_down_sync(0xffffffffu, s, o);
    s2 += __shfl_down_sync(0xffffffffu, s2, o);
  }
  if ((threadIdx.x & 31) == 0 && acc) {
    atomicAdd(&acc[0], s);
    atomicAdd(&acc[1], s2);
  }
}

// columns [start, start + n_col) of the x dimension, wrapping around
__global__ void __launch_bounds__(256)
    resetColsKernel(float *w, const float4 *par4, const float4 *par3, int x_size, int d_size,
                    int start_col, int n_col, float reset_prob, float reset_std, PhiloxKey key,
                    uint32_t call) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= (long long)n_col * d_size) {
    return;
  }
  const int jc = (int)(t / d_size), i = (int)(t % d_size);
  const int j = (start_col + jc) % x_size;
  const long long e = (long long)j * d_size + i;
  uint32_t r[4];
  philox4x32_10((uint32_t)e, (uint32_t)(e >> 32), call, TAG_RESET, key, r);
  if (reset_prob < 1.0f && !(u01(r[0]) < reset_prob)) {
    return;
  }
  float z0, z1;
  boxMuller(r[1], r[2], z0, z1);
  float v = reset_std > 0.0f ? reset_std * z0 : 0.0f;
  if (par4) {
    const float4 q = par4[e];
    v += par3[e].z;
    v = fminf(v, q.z);
    v = fmaxf(v, q.w);
  }
  w[e] = v;
}

__global__ void __launch_bounds__(256)
    uniformInitKernel(float *w, long long n, float lo, float hi, PhiloxKey key, uint32_t call) {
  const long long t4 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t4 * 4 >= n) {
    return;
  }
  uint32_t r[4];
  philox4x32_10((uint32_t)t4, (uint32_t)(t4 >> 32), call, TAG_UNIFORM_INIT, key, r);
  for (int k = 0; k < 4; k++) {
    const long long t = t4 * 4 + k;
    if (t < n) {
      w[t] = lo + (hi - lo) * u01(r[k]);
    }
  }
}

inline unsigned blocksFor(long long n) { return (unsigned)((n + 255) / 256); }

} // namespace

void Tile::requireSingleDevice(const char *what) {
  requireDevice(what);
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    AB200_FATAL(what << " is not implemented for compound (Transfer) devices");
  }
}

// decay scale, diffusion rate and reset bias per element, uploaded on first use
// The weight matrices a weight operation acts on, each with its device: the weights of a single
// device; for a Transfer compound the fast tile with device 0 and the visible (slow) tile with
// device 1, one after the other (TransferRPUDevice::decayWeights ... with a fully hidden fast tile,
// rpu_transfer_device.cpp:612-638: the last device acts on the visible weights).
int Tile::opTargets(float *w[2], DeviceStore *ds[2]) {
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    w[0] = w_fast_;
    ds[0] = &dev_[0];
    w[1] = w_;
    ds[1] = &dev_[1];
    return 2;
  }
  w[0] = w_;
  ds[0] = &dev_[0];
  return 1;
}

void Tile::ensurePar3(DeviceStore &ds) {
  if (ds.kind == AB200_DEVICE_IDEAL || ds.par3_valid) {
    return;
  }
  const size_t size = (size_t)x_size_ * d_size_;
  const float *decay = &ds.host[4 * size], *diff = &ds.host[5 * size], *rb = &ds.host[6 * size];
  std::vector<float4> p3(size);
  for (int i = 0; i < d_size_; i++) {
    for (int j = 0; j < x_size_; j++) {
      const size_t src = (size_t)i * x_size_ + j, dst = (size_t)j * d_size_ + i;
      p3[dst] = make_float4(decay[src], diff[src], rb[src], 0.0f);
    }
  }
  if (!ds.par3) {
    AB200_CUDA(cudaMalloc(&ds.par3, size * sizeof(float4)));
  }
  AB200_CUDA(cudaMemcpy(ds.par3, p3.data(), size * sizeof(float4), cudaMemcpyHostToDevice));
  ds.par3_valid = true;
}

void Tile::modifyWeights(const ab200_weight_modifier_params &par, cudaStream_t s) {
  requireDevice("modify_weights");
  if (par.type < AB200_WMOD_COPY || par.type > AB200_WMOD_PROG_NOISE || par.type == AB200_WMOD_PCM_NOISE) {
    AB200_FATAL("Requested WeightModifierType not implemented");
  }
  if (par.n_coeffs < 0 || par.n_coeffs > AB200_WMOD_MAX_COEFFS) {
    AB200_FATAL("modify_weights: at most " << AB200_WMOD_MAX_COEFFS << " polynomial coefficients");
  }
  const long long n = (long long)x_size_ * d_size_;
  if (!fb_w_) {
    AB200_CUDA(cudaMalloc(&fb_w_, n * sizeof(float)));
    AB200_CUDA(cudaMalloc(&fb_amax_, sizeof(float)));
  }
  // the last input column is the tail of the [x_size][d_size] layout
  const long long n_mod = par.copy_last_column ? (long long)(x_size_ - 1) * d_size_ : n;
  const bool measured = par.rel_to_actual_wmax && par.type != AB200_WMOD_COPY;
  if (measured) {
    AB200_CUDA(cudaMemsetAsync(fb_amax_, 0, sizeof(float), s));
    if (n_mod > 0) {
      const long long blocks = std::min<long long>((n_mod + 255) / 256, 1184);
      absMaxKernel<<<(unsigned)blocks, 256, 0, s>>>(w_, n_mod, reinterpret_cast<unsigned int *>(fb_amax_));
      AB200_LAUNCH_CHECK();
    }
  }
  ModifyArgs g;
  g.type = par.type;
  g.sto_round = par.sto_round;
  g.n_coeffs = par.n_coeffs;
  g.std_dev = par.std_dev;
  g.res = par.res;
  g.dorefa_clip = par.dorefa_clip;
  g.pdrop = par.pdrop;
  g.amax = par.assumed_wmax;
  g.g_max = par.g_max;
  for (int k = 0; k < AB200_WMOD_MAX_COEFFS; k++) {
    g.coeffs[k] = k < par.n_coeffs ? par.coeffs[k] : 0.0f;
  }
  modifyKernel<<<blocksFor(n), 256, 0, s>>>(w_, fb_w_, n, n_mod,
                                           measured ? reinterpret_cast<unsigned int *>(fb_amax_) : nullptr,
                                           g, key_, op_calls_++);
  AB200_LAUNCH_CHECK();
  fb_active_ = true;
  fb_in_test_ = par.enable_during_test != 0;
  fb_version_++;
}

void Tile::driftWeights(float time_since_last_call, cudaStream_t s) {
  requireSingleDevice("drift_weights");
  const long long n = (long long)x_size_ * d_size_;
  const bool ideal = dev_[0].kind == AB200_DEVICE_IDEAL;
  const ab200_drift_params &d = cfg_.device[0].drift;
  if (!ideal && !(d.nu > 0.0f)) {
    return; // a pulsed device without drift has no drifter (rpu_simple_device.cpp:118-122)
  }
  const float t0 = d.t0 > 0.0f ? d.t0 : 1.0f;
  if (!drift_prev_) {
    // WeightDrifter::initialize (weight_drifter.cpp:42-55): all clocks start now
    AB200_CUDA(cudaMalloc(&drift_prev_, n * sizeof(float)));
    AB200_CUDA(cudaMalloc(&drift_w0_, n * sizeof(float)));
    AB200_CUDA(cudaMalloc(&drift_t_, n * sizeof(float)));
    AB200_CUDA(cudaMemcpyAsync(drift_prev_, w_, n * sizeof(float), cudaMemcpyDeviceToDevice, s));
    AB200_CUDA(cudaMemcpyAsync(drift_w0_, w_, n * sizeof(float), cudaMemcpyDeviceToDevice, s));
    AB200_CUDA(cudaMemsetAsync(drift_t_, 0, n * sizeof(float), s));
    drift_now_ = 0.0f;
    if (!ideal) {
      // the exponents of the elements, in the weights' layout [x][d]; the ideal device drifts with
      // one exponent for all weights
      const size_t size = (size_t)n;
      const float *nu = &dev_[0].host[7 * size];
      std::vector<float> nt(size);
      for (int i = 0; i < d_size_; i++) {
        for (int j = 0; j < x_size_; j++) {
          nt[(size_t)j * d_size_ + i] = nu[(size_t)i * x_size_ + j];
        }
      }
      AB200_CUDA(cudaMalloc(&drift_nu_, size * sizeof(float)));
      AB200_CUDA(cudaMemcpyAsync(drift_nu_, nt.data(), size * sizeof(float), cudaMemcpyHostToDevice, s));
      AB200_CUDA(cudaStreamSynchronize(s)); // the staging vector goes out of scope
    }
  }
  drift_now_ += time_since_last_call / t0;
  DriftArgs g;
  g.nu = d.nu;
  g.nu_std = d.nu_std;
  g.wg_ratio = d.wg_ratio != 0.0f ? d.wg_ratio : 1.0f;
  g.g_offset = d.g_offset;
  g.w_offset = d.w_offset;
  g.nu_k = d.nu_k;
  g.log_g0 = d.log_g0;
  g.reset_tol = d.reset_tol > 0.0f ? d.reset_tol : 1e-7f;
  g.w_read_std = d.w_read_std;
  g.a = g.g_offset * g.wg_ratio + g.w_offset;
  if (fabsf(g.a) < g.reset_tol) {
    g.a = 0.0f;
  }
  driftKernel<<<blocksFor(n), 256, 0, s>>>(w_, drift_prev_, drift_w0_, drift_t_,
                                          drift_nu_,
                                          ideal ? nullptr : dev_[0].par4, n, drift_now_, g, key_,
                                          op_calls_++);
  AB200_LAUNCH_CHECK();
  w_version_++;
}

void Tile::decayWeights(float alpha, bool bias_no_decay, cudaStream_t s) {
  requireDevice("decay_weights");
  const long long n = (long long)x_size_ * d_size_;
  const long long first_bias = bias_no_decay ? (long long)(x_size_ - 1) * d_size_ : n;
  if (dev_[0].kind == AB200_DEVICE_IDEAL) {
    const float lifetime = cfg_.device[0].lifetime;
    const float rate = lifetime > 1.0f ? 1.0f / lifetime : 0.0f;
    const float scale = 1.0f - alpha * rate;
    if (scale > 0.0f && scale < 1.0f) {
      scaleKernel<<<blocksFor(n), 256, 0, s>>>(w_, n, first_bias, scale);
      AB200_LAUNCH_CHECK();
      w_version_++;
    }
    return;
  }
  float *w[2];
  DeviceStore *ds[2];
  const int nt = opTargets(w, ds);
  for (int k = 0; k < nt; k++) {
    ensurePar3(*ds[k]);
    decayKernel<<<blocksFor(n), 256, 0, s>>>(w[k], ds[k]->par4, ds[k]->par3, n, first_bias, alpha, 1);
    AB200_LAUNCH_CHECK();
  }
  w_version_++;
}

void Tile::diffuseWeights(cudaStream_t s) {
  requireDevice("diffuse_weights");
  const long long n = (long long)x_size_ * d_size_;
  const bool ideal = dev_[0].kind == AB200_DEVICE_IDEAL;
  if (ideal && !(cfg_.device[0].diffusion > 0.0f)) {
    return;
  }
  float *w[2];
  DeviceStore *ds[2];
  const int nt = opTargets(w, ds);
  for (int k = 0; k < nt; k++) {
    if (!ideal) {
      ensurePar3(*ds[k]);
    }
    diffuseKernel<<<blocksFor((n + 3) / 4), 256, 0, s>>>(w[k], ideal ? nullptr : ds[k]->par4,
                                                        ideal ? nullptr : ds[k]->par3, n,
                                                        cfg_.device[0].diffusion, key_, op_calls_++);
    AB200_LAUNCH_CHECK();
  }
  w_version_++;
}

void Tile::clipWeights(int type, float fixed_value, float sigma, cudaStream_t s) {
  requireDevice("clip_weights");
  const long long n = (long long)x_size_ * d_size_;
  const bool ideal = dev_[0].kind == AB200_DEVICE_IDEAL;
  const float4 *bounds = ideal ? nullptr : dev_[0].par4;
  float clip = -1.0f;
  if (type == AB200_CLIP_NONE) {
    return;
  } else if (type == AB200_CLIP_FIXED_VALUE) {
    clip = fixed_value;
    if (ideal && clip < 0.0f) {
      return; // RPUSimple::clipWeights: nothing to do without a value
    }
  } else if (type == AB200_CLIP_LAYER_GAUSSIAN || type == AB200_CLIP_AVERAGE_CHANNEL_MAX) {
    if (!ideal) {
      // rpu_pulsed.cpp:269-279
      AB200_FATAL("Sophisticated clipping is NOT implemented for most training devices");
    }
    // one statistics pass, read back: the clip value is a scalar the host needs anyway
    // statistics buffer of the tile, allocated once: two doubles + one word per output row
    if (!clip_stats_) {
      AB200_CUDA(cudaMalloc(&clip_stats_, 2 * sizeof(double) + (size_t)d_size_ * sizeof(unsigned int)));
    }
    double *acc = reinterpret_cast<double *>(clip_stats_);
    unsigned int *rowmax = nullptr;
    AB200_CUDA(cudaMemsetAsync(acc, 0, 2 * sizeof(double), s));
    if (type == AB200_CLIP_AVERAGE_CHANNEL_MAX) {
      rowmax = reinterpret_cast<unsigned int *>(clip_stats_ + 2 * sizeof(double));
      AB200_CUDA(cudaMemsetAsync(rowmax, 0, (size_t)d_size_ * sizeof(unsigned int), s));
    }
    clipStatsKernel<<<blocksFor(n), 256, 0, s>>>(w_, n, d_size_, acc, rowmax);
    AB200_LAUNCH_CHECK();
    double h[2];
    AB200_CUDA(cudaMemcpyAsync(h, acc, sizeof(h), cudaMemcpyDeviceToHost, s));
    std::vector<float> hmax;
    if (rowmax) {
      hmax.resize(d_size_);
      AB200_CUDA(cudaMemcpyAsync(hmax.data(), rowmax, (size_t)d_size_ * sizeof(float),
                                 cudaMemcpyDeviceToHost, s));
    }
    AB200_CUDA(cudaStreamSynchronize(s));
    if (type == AB200_CLIP_LAYER_GAUSSIAN) {
      const double mean = h[0] / (double)n;
      const double var = n > 1 ? (h[1] - (double)n * mean * mean) / (double)(n - 1) : 0.0;
      clip = (float)(std::sqrt(var > 0.0 ? var : 0.0) * (double)sigma);
    } else {
      double sum = 0.0;
      for (float v : hmax) {
        sum += v;
      }
      clip = (float)std::fabs(sum / (double)d_size_);
    }
    if (fixed_value > 0.0f) {
      clip = clip < fixed_value ? clip : fixed_value;
    }
    if (!(clip > 0.0f)) {
      return;
    }
  } else {
    AB200_FATAL("Clipping type not implemented.");
  }
  float *w[2];
  DeviceStore *ds[2];
  const int nt = opTargets(w, ds);
  for (int k = 0; k < nt; k++) {
    clipBoundsKernel<<<blocksFor(n), 256, 0, s>>>(w[k], ideal ? bounds : ds[k]->par4, n, clip);
    AB200_LAUNCH_CHECK();
  }
  w_version_++;
}

void Tile::resetColumns(int start_col, int n_cols, float reset_prob, cudaStream_t s) {
  requireDevice("reset_columns");
  if (reset_prob == 0.0f) {
    return; // rpu_pulsed.cpp:219-224
  }
  int n_col = n_cols >= 0 ? n_cols : x_size_;
  n_col = n_col > x_size_ ? x_size_ : n_col;
  if (n_col == 0) {
    return;
  }
  if (start_col < 0 || start_col >= x_size_) {
    AB200_FATAL("reset_columns: start column " << start_col << " outside [0, " << x_size_ << ")");
  }
  const bool ideal = dev_[0].kind == AB200_DEVICE_IDEAL;
  float *w[2];
  DeviceStore *ds[2];
  // a Transfer compound resets its fast tile only (rpu_transfer_device.cpp:646-651)
  const int nt = cfg_.device_kind == AB200_DEVICE_TRANSFER ? (opTargets(w, ds), 1) : opTargets(w, ds);
  for (int k = 0; k < nt; k++) {
    if (!ideal) {
      ensurePar3(*ds[k]);
    }
    const float reset_std = ideal ? cfg_.device[0].reset_std : ds[k]->reset_std;
    resetColsKernel<<<blocksFor((long long)n_col * d_size_), 256, 0, s>>>(
        w[k], ideal ? nullptr : ds[k]->par4, ideal ? nullptr : ds[k]->par3, x_size_, d_size_,
        start_col, n_col, reset_prob, reset_std, key_, op_calls_++);
    AB200_LAUNCH_CHECK();
  }
  w_version_++;
}

void Tile::setWeightsUniformRandom(float lo, float hi, cudaStream_t s) {
  requireSingleDevice("set_weights_uniform_random");
  const long long n = (long long)x_size_ * d_size_;
  uniformInitKernel<<<blocksFor((n + 3) / 4), 256, 0, s>>>(w_, n, lo, hi, key_, op_calls_++);
  AB200_LAUNCH_CHECK();
  if (dev_[0].kind != AB200_DEVICE_IDEAL) {
    // onSetWeights: clip to the per-element bounds (rpu_pulsed.cpp:280-284)
    clipBoundsKernel<<<blocksFor(n), 256, 0, s>>>(w_, dev_[0].par4, n, -1.0f);
    AB200_LAUNCH_CHECK();
  }
  w_version_++;
}

} // namespace ab200
