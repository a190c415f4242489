// Per-element steps of the IO-managed MVM, shared by the CUDA-core and tensor-core kernels.
// Every step is written with explicit round-to-nearest fp32 intrinsics so that the compiler
// cannot contract them into FMAs: the reference CPU build has no fused multiply-adds
// (CMakeLists.txt:52-53) and a 1-ulp difference in front of rint() can move a DAC/ADC code.
#pragma once

#include "common.cuh"
#include "tile.h"

namespace ab200 {

// element k of gathered row r (RowGather, tile.h)
__device__ __forceinline__ float gatherRowElement(const RowGather &g, const float *images, int r, int k) {
  const int n = r / g.m_batch, l = r - n * g.m_batch;
  const int j = __ldg(g.idx + (long long)l * g.ld + k);
  return j <= 1 ? (float)j : __ldg(images + (long long)n * g.image_size + (j - 2));
}

// address of output (row r, column n) of an MVM: strided, or transposed in blocks of rows
__device__ __forceinline__ float *mvmOutPtr(const MvmProblem &p, int r, int n) {
  if (p.out_t_rows > 0) {
    const int blk = r / p.out_t_rows, l = r - blk * p.out_t_rows;
    return p.out + ((long long)blk * p.out_size + n) * p.out_t_rows + l;
  }
  return p.out + (long long)r * p.out_ss + (long long)n * p.out_fs;
}

// Per-sample statistics of the raw input that the noise-management types need.
struct NmStats {
  float amax = 0.0f;      // max |x|
  float vmax = -3.4e38f;  // max x
  float psum = 0.0f;      // sum of the positive inputs
  float nsum = 0.0f;      // sum of the negative inputs
  __device__ __forceinline__ void add(float x) {
    amax = fmaxf(amax, fabsf(x));
    vmax = fmaxf(vmax, x);
    psum += x > 0.0f ? x : 0.0f;
    nsum += x < 0.0f ? x : 0.0f;
  }
  __device__ __forceinline__ void warpReduce() {
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      psum += __shfl_xor_sync(0xffffffffu, psum, o);
      nsum += __shfl_xor_sync(0xffffffffu, nsum, o);
    }
  }
};

// AbsMaxNPSum (rpu_forward_backward_pass.cpp:152-173): the larger of the abs-max and a bound on
// the output, sum of the same-sign inputs times the assumed largest weight over the output bound.
__device__ __forceinline__ float nmValueNPSum(const IOEff &io, const NmStats &st) {
  const float bound = isinf(io.out_bound) ? 1.0f : io.out_bound;
  const float sum = fmaxf(st.psum, -st.nsum);
  const float amax = io.nm_thres > 0.0f ? fminf(st.amax, io.nm_thres) : st.amax;
  float np = __fdiv_rn(__fmul_rn(sum, io.nm_assumed_wmax), bound);
  if (io.res_in > 0.0f) {
    np = fminf(__fmul_rn(__fdiv_rn(amax, io.res_in), io.max_bm_res), np);
  }
  return fmaxf(amax, np);
}

// computeNoiseManagement (src/rpucuda/rpu_forward_backward_pass.cpp:113-178)
__device__ __forceinline__ bool nmNeedsStats(const IOEff &io) {
  return !io.is_perfect && (io.nm == AB200_NM_ABS_MAX || io.nm == AB200_NM_MAX ||
                            io.nm == AB200_NM_ABS_MAX_NP_SUM);
}
__device__ __forceinline__ float nmValue(const IOEff &io, const NmStats &st) {
  if (io.is_perfect) {
    return 1.0f;
  }
  switch (io.nm) {
  case AB200_NM_ABS_MAX:
    return io.nm_thres > 0.0f ? fminf(st.amax, io.nm_thres) : st.amax;
  case AB200_NM_MAX:
    return io.nm_thres > 0.0f ? fminf(st.vmax, io.nm_thres) : st.vmax;
  case AB200_NM_ABS_MAX_NP_SUM:
    return nmValueNPSum(io, st);
  case AB200_NM_CONSTANT:
    return io.nm_thres > 0.0f ? io.nm_thres : 1.0f;
  default:
    return 1.0f;
  }
}
__device__ __forceinline__ float nmValue(const IOEff &io, float amax) {
  NmStats st;
  st.amax = amax;
  return nmValue(io, st);
}

// Input scale of one sample; 0 marks "output is identically zero"
// (forward: rpu_forward_backward_pass.cpp:924-969; backward: :1003-1022).
__device__ __forceinline__ float
inputScale(const IOEff &io, float sval, float reduction, bool forward) {
  if (io.is_perfect) {
    return 1.0f;
  }
  bool nm = io.nm != AB200_NM_NONE;
  if (nm && sval <= 0.0f) {
    if (!(forward && io.inp_noise > 0.0f)) {
      return 0.0f;
    }
    nm = false; // forward with input noise goes on without the input scaling (:924, :960-963)
  }
  float scale = 1.0f;
  if (nm) {
    scale = __fdiv_rn(1.0f, sval);
  }
  if (forward && io.bm != AB200_BM_NONE) {
    scale = __fdiv_rn(scale, reduction);
  }
  return scale;
}

// Random numbers of one input element: a pure function of (sample, feature, call, tag), so every
// kernel that prepares the same element (norm of the inputs, product, bound-management re-run of
// the same round) sees the same draw.
struct ElemRng {
  PhiloxKey key;
  uint32_t call;
  uint32_t tag; // TAG_FWD_IN / TAG_BWD_IN + tile id + round
};
__device__ __forceinline__ bool inputIsRandom(const IOEff &io) {
  return !io.is_perfect && (io.inp_noise > 0.0f || (io.inp_sto_round && io.res_in > 0.0f));
}

// getDiscretizedValue with sto_round (src/rpucuda/utility_functions.h:186-193):
// rint(v / res + (u - 0.5)) * res
__device__ __forceinline__ float discretizeSto(float v, float res, float u) {
  return res > 0.0f ? __fmul_rn(rintf(__fadd_rn(__fdiv_rn(v, res), __fadd_rn(u, -0.5f))), res) : v;
}

// prepareInputImplStage4 (rpu_forward_backward_pass.cpp:571-604): scale, DAC (rounding to nearest
// or stochastic), clip, input noise (after the clip, as there), asymmetry of negative values.
__device__ __forceinline__ float
prepareInput(const IOEff &io, float x, float scale, const ElemRng &g, uint32_t sample, uint32_t k) {
  if (io.is_perfect) {
    return x;
  }
  float v = __fmul_rn(x, scale);
  if (inputIsRandom(io)) {
    uint32_t r[4];
    philox4x32<7>(k, sample, g.call, g.tag, g.key, r);
    v = io.inp_sto_round ? discretizeSto(v, io.res_in, u01(r[0])) : discretize(v, io.res_in);
    v = v > io.inp_bound ? io.inp_bound : v;
    v = v < -io.inp_bound ? -io.inp_bound : v;
    if (io.inp_noise > 0.0f) {
      float z0, z1;
      boxMuller(r[1], r[2], z0, z1);
      v = __fadd_rn(v, __fmul_rn(io.inp_noise, z0));
    }
  } else {
    v = discretize(v, io.res_in);
    v = v > io.inp_bound ? io.inp_bound : v;
    v = v < -io.inp_bound ? -io.inp_bound : v;
  }
  if (io.inp_asym != 1.0f) {
    v = v < 0.0f ? __fmul_rn(v, io.inp_asym) : v;
  }
  return v;
}
// the plain DAC (no random part, no asymmetry): read-out of a transfer
__device__ __forceinline__ float prepareInput(const IOEff &io, float x, float scale) {
  if (io.is_perfect) {
    return x;
  }
  float v = discretize(__fmul_rn(x, scale), io.res_in);
  v = v > io.inp_bound ? io.inp_bound : v;
  v = v < -io.inp_bound ? -io.inp_bound : v;
  return v;
}

// Std-dev of the Gaussian added before the ADC: output noise (:695-698) and the additive-constant
// weight noise w_noise * ||v|| (:341-352) are independent zero-mean Gaussians on the same value,
// so one draw with the combined variance is statistically identical to two draws.
__device__ __forceinline__ float outputSigma(const IOEff &io, float vnorm) {
  float s = io.out_noise;
  if (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f) {
    float ws = io.w_noise * vnorm;
    s = sqrtf(s * s + ws * ws);
  }
  return s;
}

// The same with the two extensions of the CUDA-core kernels: a std-dev of the output noise per
// output line (`onv`, rpu_forward_backward_pass.cpp:306-313, :696) and the PCMRead weight noise
// w_noise * sqrt(sum_j |w_ij| v_j^2) (:353-381), `pcm` being that sum for the element.
__device__ __forceinline__ float
outputSigmaLine(const IOEff &io, float vnorm, const float *onv, int col, float pcm) {
  float s = onv ? onv[col] : io.out_noise;
  if (io.w_noise > 0.0f) {
    if (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT) {
      float ws = io.w_noise * vnorm;
      s = sqrtf(s * s + ws * ws);
    } else if (io.w_noise_type == AB200_WNOISE_PCM_READ) {
      s = sqrtf(s * s + io.w_noise * io.w_noise * pcm);
    }
  }
  return s;
}
__host__ __device__ __forceinline__ bool ioLineSigma(const IOEff &io) {
  return io.out_noise_std > 0.0f || (io.w_noise_type == AB200_WNOISE_PCM_READ && io.w_noise > 0.0f);
}
// IO settings that need the extra accumulators and the long output chain of the CUDA-core kernels
__host__ __device__ __forceinline__ bool ioNeedsLineChain(const IOEff &io) {
  return !io.is_perfect &&
         ((io.w_noise_type == AB200_WNOISE_PCM_READ && io.w_noise > 0.0f) || io.ir_drop > 0.0f ||
          io.v_offset_std > 0.0f || io.r_series > 0.0f || io.out_nl > 0.0f || io.pos_neg != 0);
}

// Weight of input position k in the IR-drop term: 1 - (1 - k / n)^2
// (rpu_forward_backward_pass.cpp:418-422)
__device__ __forceinline__ float irPosWeight(int k, int n) {
  const float p = __fsub_rn(1.0f, __fdiv_rn((float)k, (float)n));
  return __fsub_rn(1.0f, __fmul_rn(p, p));
}

// The analog output of one line before the ADC stage, with the non-idealities in the reference's
// order (applyNonIdealities + finalizeOutput, rpu_forward_backward_pass.cpp:540-566, :673-719):
// IR drop, voltage offset / series resistance, weight noise, output non-linearity. `cur` =
// sum |w| |v|, `irsum` = sum w v posw, `pcm` = sum |w| v^2 of the line; z_w a standard normal.
struct LineChain {
  const float *v_offset;
  const float *out_nl;
  float nl_factor;
  float a_scale; // in_size / ir_drop_g_ratio
};
// The output non-linearity of a line: first step of the output stage (finalizeOutput :673-719)
__device__ __forceinline__ float lineNonLinearity(const LineChain &lc, float y, int col) {
  if (lc.out_nl) {
    y = __fdiv_rn(__fmul_rn(lc.nl_factor, y), __fadd_rn(1.0f, fabsf(__fmul_rn(lc.out_nl[col], y))));
  }
  return y;
}
// `with_nl = false` stops after the steps that belong to one pass through the array
// (applyNonIdealities); the two-pass MV types add their halves there.
__device__ __forceinline__ float lineChain(const IOEff &io, const LineChain &lc, float y, int col,
                                           float cur, float irsum, float pcm, float vnorm, float z_w,
                                           bool with_nl = true) {
  if (io.ir_drop > 0.0f) {
    const float a = __fmul_rn(lc.a_scale, cur);
    const float c = __fmul_rn(a, __fadd_rn(__fmul_rn(a, __fsub_rn(__fmul_rn(0.05f, a), 0.2f)), 0.5f));
    y = __fsub_rn(y, __fmul_rn(c, __fmul_rn(io.ir_drop, irsum)));
  }
  if (lc.v_offset) {
    const float vo = lc.v_offset[col];
    if (io.r_series > 0.0f) {
      const float nom = __fadd_rn(1.0f, fminf(__fmul_rn(io.r_series, fabsf(y)), io.r_series_max));
      y = __fdiv_rn(__fmul_rn(__fsub_rn(1.0f, vo), y), nom);
    } else {
      y = __fmul_rn(y, __fsub_rn(1.0f, vo));
    }
  }
  if (io.w_noise > 0.0f) {
    if (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT) {
      y = __fadd_rn(y, __fmul_rn(__fmul_rn(io.w_noise, vnorm), z_w));
    } else if (io.w_noise_type == AB200_WNOISE_PCM_READ) {
      y = __fadd_rn(y, __fmul_rn(__fmul_rn(io.w_noise, sqrtf(pcm)), z_w));
    }
  }
  return with_nl ? lineNonLinearity(lc, y, col) : y;
}

// four uniforms in (0,1) for the stochastic ADC rounding of noise block `blk` (four output columns)
__device__ __forceinline__ void
uniform4(PhiloxKey key, uint64_t blk, uint32_t call, uint32_t tag, float u[4]) {
  uint32_t r[4];
  philox4x32<7>((uint32_t)blk, (uint32_t)(blk >> 32), call, tag, key, r);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    u[j] = u01(r[j]);
  }
}

// finalizeOutputImplStage5 (rpu_forward_backward_pass.cpp:673-719): asymmetry of negative values,
// noise, ADC (rounding to nearest, or stochastic with the uniform `u`), clip / bound test.
__device__ __forceinline__ float
finalizeOutput(const IOEff &io, float y, float sigma, float z, bool &exceeded, float u = 0.5f) {
  if (io.out_asym != 1.0f) {
    y = y < 0.0f ? __fmul_rn(y, io.out_asym) : y;
  }
  if (sigma > 0.0f) {
    y = __fadd_rn(y, __fmul_rn(sigma, z));
  }
  y = io.out_sto_round ? discretizeSto(y, io.res_out, u) : discretize(y, io.res_out);
  if (y > io.out_bound) {
    y = io.out_bound;
    exceeded = true;
  } else if (y < -io.out_bound) {
    y = -io.out_bound;
    exceeded = exceeded || (io.bm_test_negative_bound != 0);
  }
  return y;
}

// Final rescale: forward out_scale*alpha/scale (:985-987), backward out_scale*alpha*s (:1024-1026).
__device__ __forceinline__ float
outputFactor(const IOEff &io, float alpha, float sval, float scale, bool backward) {
  float os = __fmul_rn(io.out_scale, alpha);
  if (io.is_perfect) {
    return os;
  }
  if (scale == 0.0f) {
    return 0.0f;
  }
  return backward ? __fmul_rn(os, sval) : __fdiv_rn(os, scale);
}

} // namespace ab200
