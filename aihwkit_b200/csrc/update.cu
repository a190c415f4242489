// Pulsed weight update.
//
//   pulsePrepareKernel   per sample: |x|max, |d|max -> BL, A, B (update management), then the pulse
//                        train of every x- and d-line packed into one 32-bit word (bit 0 = sign,
//                        bits 1..BL = pulses), or the implicit pulse values for the deterministic
//                        pulse type.
//   pulsedUpdateKernel   per weight element: coincidences by AND + popc over the batch, device
//                        rule applied pulse by pulse in place; weights and per-element parameters
//                        are read with coalesced 128-bit loads, once per call.
//
// Reference semantics restated here:
//   update management      src/rpucuda/rpu_pulsed_meta_parameter.cpp:153-236
//   stochastic trains      src/rpucuda/sparse_bit_line_maker.cpp:200-238, 288-353
//   implicit pulses        src/rpucuda/dense_bit_line_maker.cpp:210-264
//   coincidence loop       src/rpucuda/rpu_weight_updater.cpp:236-291
//   ConstantStep           src/rpucuda/rpu_constantstep_device.cpp:28-78
//   LinearStep/SoftBounds  src/rpucuda/rpu_linearstep_device.cpp:113-164
//   SoftBoundsReference    src/rpucuda/rpu_softbounds_reference_device.cpp:107-175
#include "mvm_common.cuh"
#include "tile.h"

namespace ab200 {

__device__ __forceinline__ float blockMax(float v, float *sh) {
  for (int o = 16; o > 0; o >>= 1) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  }
  int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    sh[w] = v;
  }
  __syncthreads();
  float r = 0.0f;
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) {
    r = fmaxf(r, sh[i]);
  }
  __syncthreads();
  return r;
}

// calculateBlAB + performUpdateManagement, fp32 with the reference's association
// (rpu_pulsed_meta_parameter.cpp:153-236). BL == 0 means "no update for this sample".
__device__ __forceinline__ void
blAB(const UpEff &up, float lr, float dw_min, float xm, float dm, int &BL, float &A, float &B) {
  if (lr == 0.0f) {
    BL = 0;
    A = B = 0.0f;
    return;
  }
  if (up.fixed_bl || up.update_bl_management) {
    BL = up.desired_bl;
    A = __fsqrt_rn(__fdiv_rn(lr, __fmul_rn(dw_min, (float)BL)));
    B = A;
  } else {
    if (__fmul_rn(dw_min, (float)up.desired_bl) < lr) {
      A = B = 1.0f;
      BL = max((int)ceilf(__fdiv_rn(lr, dw_min)), 1);
    } else {
      BL = up.desired_bl;
      A = __fsqrt_rn(__fdiv_rn(lr, __fmul_rn(dw_min, (float)BL)));
      B = A;
    }
  }
  if (up.update_bl_management || up.update_management) {
    if (xm == 0.0f || dm == 0.0f) {
      BL = 0;
      A = B = 1.0f;
      return;
    }
    float x_val = xm;
    float d_val = __fmul_rn(up.um_grad_scale, dm);
    float k_val = __fdiv_rn(__fmul_rn(__fmul_rn(lr, x_val), d_val), dw_min);
    if (up.update_bl_management) {
      BL = (int)ceilf(k_val);
      if (BL > up.desired_bl) {
        BL = up.desired_bl;
      }
      A = __fsqrt_rn(__fdiv_rn(lr, __fmul_rn(dw_min, (float)BL)));
      B = A;
    }
    if (up.update_management) {
      if (k_val > (float)up.desired_bl) {
        d_val = __fmul_rn(d_val, __fdiv_rn((float)up.desired_bl, k_val));
      }
      A = __fmul_rn(A, __fsqrt_rn(__fdiv_rn(x_val, d_val)));
      B = __fmul_rn(B, __fsqrt_rn(__fdiv_rn(d_val, x_val)));
    }
  }
}

// One stochastic pulse train (generateCounts, sparse_bit_line_maker.cpp:200-238): BL Bernoulli
// draws with probability pp; each draw compares pp against a 16-bit uniform, 8 draws per
// Philox call. (A bit-serial comparison of all slots at once - one random word per bit of pp until
// every slot is decided - needs fewer calls per lane but as many per warp, and measured slower.)
__device__ __forceinline__ uint32_t
pulseTrain(float pp, int BL, int seg, PhiloxKey key, uint32_t line, uint32_t sample, uint32_t call,
           uint32_t tag) {
  // slots [seg * 31, min(BL, seg * 31 + 31)) of the train, as bits 1.. of one word
  const int k0 = seg * kPulseSegSlots;
  const int nk = min(BL - k0, kPulseSegSlots);
  float thr = pp * 65536.0f;
  uint32_t bits = 0;
  int k = 0;
  for (int q = 0; q * 8 < nk; q++) {
    uint32_t r[4];
    philox4x32<7>(line, sample, call, tag + (uint32_t)(seg * 4 + q), key, r);
#pragma unroll
    for (int h = 0; h < 8; h++) {
      uint32_t u16 = (r[h >> 1] >> ((h & 1) * 16)) & 0xFFFFu;
      if (k < nk && ((float)u16 + 0.5f) < thr) {
        bits |= 1u << (k + 1);
      }
      k++;
    }
  }
  return bits;
}

// getDiscretizedValue of a pulse probability (src/rpucuda/utility_functions.h:186-193): to the
// nearest multiple of `res`, or - with sto_round - up or down at random in proportion to the
// remainder; the uniform of a line is a function of (line, sample, call).
__device__ __forceinline__ float
pulseProb(const UpdateProblem &p, float v, float res, uint32_t line, uint32_t sample, uint32_t tag) {
  if (!p.up.sto_round || !(res > 0.0f)) {
    return discretize(v, res);
  }
  uint32_t r[4];
  philox4x32<7>(line, sample, p.call, tag ^ 0x08000000u, p.key, r);
  return __fmul_rn(rintf(__fadd_rn(__fdiv_rn(v, res), __fadd_rn(u01(r[0]), -0.5f))), res);
}

__global__ void __launch_bounds__(256) pulsePrepareKernel(UpdateProblem p) {
  pdlEnter();
  __shared__ float sh[8];
  __shared__ float s_A, s_B;
  __shared__ int s_BL;
  const int s = blockIdx.x;
  const float *xr = p.x + (long long)s * p.x_ss;
  const float *dr = p.d + (long long)s * p.d_ss;
  const bool need_max = p.up.update_management || p.up.update_bl_management;
  // samples gathered from whole images (indexed convolution interface) or plain rows
  const bool gathered = p.gather.idx != nullptr;
  auto xValue = [&](int j) -> float {
    if (gathered) {
      return gatherRowElement(p.gather, p.x, s, j);
    }
    return j < p.x_real ? xr[(long long)j * p.x_fs] : 1.0f;
  };
  float xm = 0.0f, dm = 0.0f;
  if (need_max) {
    for (int j = threadIdx.x; j < p.x_size; j += blockDim.x) {
      xm = fmaxf(xm, fabsf(xValue(j)));
    }
    for (int i = threadIdx.x; i < p.d_size; i += blockDim.x) {
      dm = fmaxf(dm, fabsf(dr[(long long)i * p.d_fs]));
    }
    xm = blockMax(xm, sh);
    dm = blockMax(dm, sh);
  }
  if (threadIdx.x == 0) {
    int BL;
    float A, B;
    blAB(p.up, p.lr, p.dw_min, xm, dm, BL, A, B);
    s_BL = BL;
    s_A = A;
    s_B = B;
  }
  __syncthreads();
  const int BL = s_BL;
  const float A = s_A, B = s_B;
  const int nseg = p.nseg > 0 ? p.nseg : 1;
  uint32_t *xw = p.xw + (long long)s * nseg * p.x_size;
  uint32_t *dw = p.dw + (long long)s * nseg * p.d_size;
  const bool implicit = p.up.pulse_type == AB200_PULSE_DETERMINISTIC_IMPLICIT;
  const bool mean_count = p.up.pulse_type == AB200_PULSE_MEAN_COUNT;

  for (int l = threadIdx.x; l < p.x_size + p.d_size; l += blockDim.x) {
    const bool is_x = l < p.x_size;
    const int idx = is_x ? l : l - p.x_size;
    float v = is_x ? xValue(idx) : dr[(long long)idx * p.d_fs];
    const float P = is_x ? B : A;
    uint32_t word;
    if (implicit) {
      // generateDetImplicit (dense_bit_line_maker.cpp:210-238); d-values carry the factor BL
      // (generateCoincidencesDetI :240-264)
      float vv = p.lr_neg ? -v : v;
      float pp = pulseProb(p, __fmul_rn(fabsf(vv), P), is_x ? p.up.x_res_implicit : p.up.d_res_implicit,
                           (uint32_t)idx, (uint32_t)s, is_x ? TAG_PULSE_X : TAG_PULSE_D);
      pp = fmaxf(fminf(pp, 1.0f), 0.0f);
      float sv = vv >= 0.0f ? pp : -pp;
      if (BL == 0) {
        sv = 0.0f;
      }
      if (!is_x) {
        sv = __fmul_rn(sv, (float)BL);
      }
      word = __float_as_uint(sv);
    } else if (mean_count) {
      // generateCountsMean / generateCoincidences (dense_bit_line_maker.cpp:142-204): the mean
      // number of pulses per line, no fluctuation; the d count carries the factor 1 / BL, so the
      // coincidences are rint(d * x) like those of the implicit type
      const float vv = p.lr_neg ? -v : v;
      const float pp = pulseProb(p, __fmul_rn(fabsf(vv), P), p.up.res, (uint32_t)idx, (uint32_t)s,
                                 is_x ? TAG_PULSE_X : TAG_PULSE_D);
      float sv = 0.0f;
      if (pp != 0.0f && BL > 0) {
        const int ntimes = max(min((int)rintf(__fmul_rn((float)BL, pp)), BL), 0);
        sv = (vv >= 0.0f || ntimes == 0) ? (float)ntimes : -(float)ntimes;
        if (!is_x) {
          sv = __fdiv_rn(sv, (float)BL);
        }
      }
      word = __float_as_uint(sv);
    } else {
      float pp = 0.0f;
      uint32_t neg = 0u;
      if (BL > 0) {
        pp = pulseProb(p, __fmul_rn(fabsf(v), P), p.up.res, (uint32_t)idx, (uint32_t)s,
                       is_x ? TAG_PULSE_X : TAG_PULSE_D);
        neg = v > 0.0f ? 0u : 1u;
        if (!is_x && p.lr_neg) {
          neg ^= 1u;
        }

      }
      const int n_lines = is_x ? p.x_size : p.d_size;
      for (int g = 0; g < nseg; g++) {
        word = 0;
        if (pp != 0.0f && g * kPulseSegSlots < BL) {
          word = pulseTrain(pp, BL, g, p.key, (uint32_t)idx, (uint32_t)s, p.call,
                            is_x ? TAG_PULSE_X : TAG_PULSE_D);
          word = word ? (word | neg) : 0u;
        }
        (is_x ? xw : dw)[(long long)g * n_lines + idx] = word;
      }
      continue;
    }
    (is_x ? xw : dw)[idx] = word;
  }
}

// ---------------------------------------------------------------------------------------------
// device rules: one pulse, clipped immediately. `down` = weight decreases.
// par4 = {scale_up, scale_down, max_bound, min_bound}
// ---------------------------------------------------------------------------------------------
template <int KIND>
__device__ __forceinline__ float pulseOnce(float w, bool down, const float4 &q, const float2 &e,
                                           float xi, int mult_noise, const float4 &es0,
                                           const float4 &es1, const float *pw = nullptr,
                                           int pw_n = 0) {
  if (KIND == AB200_DEVICE_PIECEWISE_STEP) {
    // PiecewiseStepRPUDevice update_once (rpu_piecewisestep_device.cpp:30-80): the step factor is
    // interpolated linearly between pw_n nodes spread evenly over [min_bound, max_bound];
    // pw[0..pw_n) are the up factors, pw[pw_n..2 pw_n) the down factors
    const float *tab = down ? pw + pw_n : pw;
    const int n_sec = pw_n - 1;
    float f;
    if (n_sec <= 0 || q.z <= q.w) {
      f = __ldg(tab);
    } else {
      const float ws = fmaxf(
          __fmul_rn(__fdiv_rn(__fsub_rn(w, q.w), __fsub_rn(q.z, q.w)), (float)n_sec), 0.0f);
      const int idx = min((int)floorf(ws), n_sec - 1);
      const float t = fminf(__fsub_rn(ws, (float)idx), 1.0f);
      const float t1 = __fsub_rn(1.0f, t);
      f = __fadd_rn(__fmul_rn(t1, __ldg(tab + idx)), __fmul_rn(t, __ldg(tab + idx + 1)));
    }
    const float step = __fmul_rn(__fmul_rn(down ? q.y : q.x, f), __fadd_rn(1.0f, xi));
    w = down ? __fsub_rn(w, step) : __fadd_rn(w, step);
    w = fmaxf(w, q.w);
    w = fminf(w, q.z);
    return w;
  } else if (KIND == AB200_DEVICE_EXP_STEP) {
    // ExpStepRPUDevice update_once / update_once_complex_noise (rpu_expstep_device.cpp:18-100):
    // z = 2 w / (max - min) * a + b;  step = scale * max(1 - A exp(+-gamma z), 0)
    // es0 = {a, b, A_up, A_down}, es1 = {gamma_up, gamma_down, std_add, std_slope}; xi = std * N
    const float b_diff = __fsub_rn(q.z, q.w);
    if (!(b_diff > 0.0f)) {
      return w;
    }
    const float z = __fadd_rn(__fmul_rn(__fdiv_rn(__fmul_rn(2.0f, w), b_diff), es0.x), es0.y);
    const float y = down ? fmaxf(__fsub_rn(1.0f, __fmul_rn(es0.w, expf(__fmul_rn(es1.y, -z)))), 0.0f)
                         : fmaxf(__fsub_rn(1.0f, __fmul_rn(es0.z, expf(__fmul_rn(es1.x, z)))), 0.0f);
    if (es1.z != 0.0f || es1.w != 0.0f) {
      const float dw = down ? -__fmul_rn(y, q.y) : __fmul_rn(y, q.x);
      const float spread =
          __fadd_rn(__fadd_rn(fabsf(dw), es1.z), __fmul_rn(es1.w, fabsf(w)));
      w = __fadd_rn(w, __fadd_rn(dw, __fmul_rn(spread, xi)));
    } else {
      const float step = __fmul_rn(__fmul_rn(y, __fadd_rn(1.0f, xi)), down ? q.y : q.x);
      w = down ? __fsub_rn(w, step) : __fadd_rn(w, step);
    }
    w = fminf(w, q.z);
    w = fmaxf(w, q.w);
    return w;
  } else if (KIND == AB200_DEVICE_POW_STEP) {
    // PowStepRPUDevice update_once (rpu_powstep_device.cpp:91-121): the step shrinks with a power
    // of the distance to the bound, e = {gamma_up, gamma_down}
    const float range = __fsub_rn(q.z, q.w);
    if (range == 0.0f) {
      return w;
    }
    if (down) {
      const float f = powf(__fdiv_rn(__fsub_rn(w, q.w), range), e.y);
      w = __fsub_rn(w, __fmul_rn(__fmul_rn(q.y, f), __fadd_rn(1.0f, xi)));
    } else {
      const float f = powf(__fdiv_rn(__fsub_rn(q.z, w), range), e.x);
      w = __fadd_rn(w, __fmul_rn(__fmul_rn(q.x, f), __fadd_rn(1.0f, xi)));
    }
    w = fmaxf(w, q.w);
    w = fminf(w, q.z);
    return w;
  } else if (KIND == AB200_DEVICE_CONSTANT_STEP) {
    float dw = __fmul_rn(__fadd_rn(1.0f, xi), down ? q.y : q.x);
    w = down ? __fsub_rn(w, dw) : __fadd_rn(w, dw);
    w = fminf(w, q.z);
    w = fmaxf(w, q.w);
    return w;
  } else if (KIND == AB200_DEVICE_LINEAR_STEP) {
    float slope = down ? e.y : e.x;
    float sc = down ? q.y : q.x;
    float dw;
    if (mult_noise) {
      dw = __fmul_rn(__fadd_rn(__fmul_rn(slope, w), sc), __fadd_rn(1.0f, xi));
    } else {
      dw = __fadd_rn(__fmul_rn(slope, w), __fmul_rn(sc, __fadd_rn(1.0f, xi)));
    }
    w = down ? __fsub_rn(w, dw) : __fadd_rn(w, dw);
    w = fmaxf(w, q.w);
    w = fminf(w, q.z);
    return w;
  } else { // SOFT_BOUNDS_REFERENCE
    float ref = e.x;
    w = __fadd_rn(w, ref);
    float bound = down ? q.w : q.z;
    bool ok = down ? (bound < 0.0f) : (bound > 0.0f);
    float a = ok ? __fdiv_rn(w, bound) : 0.0f;
    float sc = down ? q.y : q.x;
    float dw;
    if (mult_noise) {
      dw = __fmul_rn(__fmul_rn(sc, __fsub_rn(1.0f, a)), __fadd_rn(1.0f, xi));
    } else {
      dw = __fmul_rn(sc, __fadd_rn(__fsub_rn(1.0f, a), xi));
    }
    w = down ? __fsub_rn(w, dw) : __fadd_rn(w, dw);
    w = fmaxf(w, q.w);
    w = fminf(w, q.z);
    return __fsub_rn(w, ref);
  }
}

constexpr int UT_I = 64; // d-lines per CTA (contiguous in memory)
constexpr int UT_J = 16; // x-lines per CTA
constexpr int UBLK = 32; // samples per block = bits of one non-zero bitmap word
constexpr int UT_JP = UT_J + 1; // padded row length of the staged x words (bank spread)

// Bitmaps of the non-empty pulse words: bit s of the word of a line is set when the pulse word of
// sample blk * 32 + s on that line carries at least one pulse (or a non-zero implicit value). The
// update kernel builds them in shared memory while it stages the words, intersects the bitmaps of
// a d-line and an x-line and only looks at the samples that survive - the GPU form of the index
// lists the reference CPU builds per pulse slot (src/rpucuda/sparse_bit_line_maker.cpp:200-238).

// Every thread owns EJ weights (one d-line, EJ x-lines; EJ = 4 with 256 threads per CTA for large
// problems, EJ = 1 with 1024 threads when the grid would otherwise not fill the GPU). The loop
// over a thread's weights is NOT unrolled: its body always works on slot 0 of the register arrays,
// which are rotated by one after every weight, so the (large) body exists once and stays in the
// instruction cache. Per super-block of 128 samples the thread
// walks, for each of its weights, the samples where both lines pulsed; the walk is decoupled from
// the (expensive, rare) pulse application: each lane first advances to ITS next coincidence, then
// the whole warp applies one event per lane together, so lanes whose events fall on different
// samples do not serialise each other. The super-block is long so that the number of events per
// lane has a small relative spread (the warp runs as many rounds as its busiest lane). Weights
// are independent, so the per-weight sample order - the only order the reference defines
// (rpu_weight_updater.cpp:243-291) - is preserved.
constexpr int USUP = 4;              // bitmap words per super-block
constexpr int USAMP = USUP * UBLK;   // samples per super-block
constexpr int URES = 8;              // Gaussians per thread in the reservoir

template <int NT, int UTJ> struct UpdateSmem {
  uint32_t sd[USAMP][UT_I];
  uint32_t sx[USAMP][(UTJ + 1)];
  uint32_t sdnz[USUP][UT_I];
  uint32_t sxnz[USUP][UTJ];
  float sz[URES][NT];
};

// Eight fresh Gaussians for one thread's column of the reservoir. Kept out of line: the refill is
// rare, and inlining it into each of the four per-weight loop bodies makes the kernel spill out of
// the instruction cache.
__device__ __noinline__ void refillReservoir(PhiloxKey key, uint32_t gid, uint32_t refills,
                                             uint32_t call, float *column, int stride) {
  float z[8];
  gauss8(key, (uint64_t)gid | ((uint64_t)refills << 32), call, TAG_DEVICE, z);
#pragma unroll
  for (int r = 0; r < URES; r++) {
    column[r * stride] = z[r];
  }
}

template <int KIND, bool IMPLICIT, bool NOISY, int EJ, int UTJ>
__global__ void __launch_bounds__(UT_I *UTJ / EJ, (UT_I * UTJ / EJ) >= 1024 ? 1 : 4)
    pulsedUpdateKernel(UpdateProblem p) {
  pdlEnter();
  constexpr int UE_J = EJ;
  constexpr int UNT = UT_I * UTJ / EJ; // threads per CTA
  extern __shared__ __align__(16) unsigned char smem_raw[];
  UpdateSmem<UNT, UTJ> &sm = *reinterpret_cast<UpdateSmem<UNT, UTJ> *>(smem_raw);
  const int ti = threadIdx.x & (UT_I - 1);
  const int tj = threadIdx.x / UT_I;
  const int i = blockIdx.x * UT_I + ti;
  const int j0 = blockIdx.y * UTJ + tj * UE_J;
  const bool i_ok = i < p.d_size;

  float w[UE_J];
  float4 q[UE_J];
  float2 e[UE_J];
  bool loaded[UE_J], dirty[UE_J];
#pragma unroll
  for (int t = 0; t < UE_J; t++) {
    loaded[t] = false;
    dirty[t] = false;
    w[t] = 0.0f;
    q[t] = make_float4(0.f, 0.f, 0.f, 0.f);
    e[t] = make_float2(0.f, 0.f);
  }
  const float std = p.dw_min_std;
  const uint32_t gid = (blockIdx.y * gridDim.x + blockIdx.x) * (uint32_t)UNT + threadIdx.x;
  uint32_t refills = 0;
  int rc = 0;

  const int b_first = p.s_begin / USAMP, b_last = (p.s_end - 1) / USAMP;
  for (int blk = b_first; blk <= b_last; blk++) {
    const int s0 = blk * USAMP;
    // bitmaps of the non-empty words of this super-block, built while the words are staged
    for (int t = threadIdx.x; t < USUP * (UT_I + UTJ); t += blockDim.x) {
      if (t < USUP * UT_I) {
        (&sm.sdnz[0][0])[t] = 0u;
      } else {
        (&sm.sxnz[0][0])[t - USUP * UT_I] = 0u;
      }
    }
    __syncthreads();
    {
      // every thread stages one fixed column of the x words and one of the d words, so the
      // loop only advances a pointer by a row; it collects the column's bitmap bits of its
      // samples in registers (the word a sample falls into is known at compile time, or one of
      // a few) and adds them to the shared bitmap at the end
      constexpr int STEP = UNT / UTJ;               // samples between two rows of a thread
      constexpr int WPS = STEP >= 32 ? STEP / 32 : 1; // bitmap words its first row can fall into
      const int jj = threadIdx.x % UTJ, sj = threadIdx.x / UTJ;
      const int gj = blockIdx.y * UTJ + jj;
      const uint32_t *src = p.xw + (long long)(s0 + sj) * p.x_size + gj;
      const long long step = (long long)STEP * p.x_size;
      uint32_t nzb[USUP];
#pragma unroll
      for (int wq = 0; wq < USUP; wq++) {
        nzb[wq] = 0u;
      }
#pragma unroll
      for (int k = 0; k < USAMP / STEP; k++, src += step) {
        const int ss = sj + STEP * k;
        const uint32_t wv = (gj < p.x_size && s0 + ss < p.m) ? *src : 0u;
        sm.sx[ss][jj] = wv;
        const bool nz = (IMPLICIT ? (wv & 0x7fffffffu) : wv) != 0u;
        const uint32_t bit = nz ? 1u << (ss & 31) : 0u;
        if (STEP < 32) {
          nzb[(STEP * k) >> 5] |= bit;
        } else {
#pragma unroll
          for (int c = 0; c < WPS; c++) {
            nzb[WPS * k + c] |= (sj >> 5) == c ? bit : 0u;
          }
        }
      }
#pragma unroll
      for (int wq = 0; wq < USUP; wq++) {
        if (nzb[wq] != 0u) {
          atomicOr(&sm.sxnz[wq][jj], nzb[wq]);
        }
      }
    }
    {
      constexpr int STEP = UNT / UT_I; // 4 or 16: a thread's rows never leave the word of STEP * k
      const int ii = threadIdx.x % UT_I, si = threadIdx.x / UT_I;
      const int gi = blockIdx.x * UT_I + ii;
      const uint32_t *src = p.dw + (long long)(s0 + si) * p.d_size + gi;
      const long long step = (long long)STEP * p.d_size;
      uint32_t nzb[USUP];
#pragma unroll
      for (int wq = 0; wq < USUP; wq++) {
        nzb[wq] = 0u;
      }
#pragma unroll
      for (int k = 0; k < USAMP / STEP; k++, src += step) {
        const int ss = si + STEP * k;
        const int sg = s0 + ss;
        const uint32_t wv = (gi < p.d_size && sg < p.m) ? *src : 0u;
        sm.sd[ss][ii] = wv;
        // samples of this super-block that belong to [s_begin, s_end): only the d bitmap needs
        // the range, a candidate needs both lines
        const bool nz = (IMPLICIT ? (wv & 0x7fffffffu) : wv) != 0u && sg >= p.s_begin && sg < p.s_end;
        nzb[(STEP * k) >> 5] |= nz ? 1u << (ss & 31) : 0u;
      }
#pragma unroll
      for (int wq = 0; wq < USUP; wq++) {
        if (nzb[wq] != 0u) {
          atomicOr(&sm.sdnz[wq][ii], nzb[wq]);
        }
      }
    }
    __syncthreads();
#pragma unroll 1
    for (int t = 0; t < UE_J; t++) {
      const int jl = tj * UE_J + t;
      const long long idx = (long long)(j0 + t) * p.d_size + i;
      // chopped transfer compound: the pulses of this weight enter with the opposite sign when
      // exactly one of its two lines is chopped (ChoppedTransferRPUDevice::doSparseUpdate /
      // doDenseUpdate, rpu_chopped_transfer_device.cpp:472-515); read per launch, so a flip by
      // a transfer between two launches of a batch takes effect for the samples after it
      bool chop_flip = false;
      if (p.chop_x != nullptr) {
        chop_flip = ((j0 + t < p.x_size ? p.chop_x[j0 + t] : 0) != 0) != ((i_ok ? p.chop_d[i] : 0) != 0);
      }
      int wi = 0;
      uint32_t cand = sm.sdnz[0][ti] & sm.sxnz[0][jl];
      while (true) {
        // advance to this lane's next coincidence
        int n = 0;
        bool down = false;
        while (true) {
          if (cand == 0u) {
            if (++wi >= USUP) {
              break;
            }
            cand = sm.sdnz[wi][ti] & sm.sxnz[wi][jl];
            continue;
          }
          const int ss = wi * UBLK + __ffs(cand) - 1;
          cand &= cand - 1u;
          const uint32_t dwv = sm.sd[ss][ti], xwv = sm.sx[ss][jl];
          if (IMPLICIT) {
            // n = rint(d * BL * x), positive = decrease (dense_bit_line_maker.cpp:240-264)
            float c = rintf(__fmul_rn(__uint_as_float(dwv), __uint_as_float(xwv)));
            n = (int)fabsf(c);
            down = (c > 0.0f) != chop_flip;
          } else {
            // coincidences of the two trains; equal line signs = decrease
            // (rpu_weight_updater.cpp:246-268)
            n = __popc((xwv & dwv) >> 1);
            down = (((xwv ^ dwv) & 1u) == 0u) != chop_flip;
          }
          if (n != 0) {
            break;
          }
        }
        if (!__any_sync(0xffffffffu, n != 0)) {
          break;
        }
        if (n != 0) {
          if (!loaded[0]) {
            w[0] = p.w[idx];
            q[0] = p.par4[idx];
            if (KIND != AB200_DEVICE_CONSTANT_STEP && KIND != AB200_DEVICE_EXP_STEP &&
                KIND != AB200_DEVICE_PIECEWISE_STEP) {
              e[0] = p.par2[idx];
            }
            loaded[0] = true;
          }
          dirty[0] = true;
        }
        if (!NOISY) {
          for (int k = 0; k < n; k++) {
            w[0] = pulseOnce<KIND>(w[0], down, q[0], e[0], 0.0f, p.mult_noise, p.es0, p.es1, p.pw, p.pw_n);
          }
        } else {
          // One Gaussian per pulse, taken from a per-thread reservoir in shared memory: the
          // generator - by far the most expensive part of a pulse - runs once per several
          // events instead of per event. The whole warp refills together as soon as one lane
          // cannot serve its event (leftovers are discarded), so the refill is never divergent;
          // only an event with more pulses than the reservoir holds refills on its own.
          if (__any_sync(0xffffffffu, n > rc)) {
            refillReservoir(p.key, gid, refills, p.call, &sm.sz[0][threadIdx.x], UNT);
            rc = URES;
            refills++;
          }
          for (int k = 0; k < n; k++) {
            if (rc == 0) {
              refillReservoir(p.key, gid, refills, p.call, &sm.sz[0][threadIdx.x], UNT);
              rc = URES;
              refills++;
            }
            rc--;
            w[0] = pulseOnce<KIND>(w[0], down, q[0], e[0], std * sm.sz[rc][threadIdx.x], p.mult_noise, p.es0,
                                    p.es1, p.pw, p.pw_n);
          }
        }
      }
      if (UE_J > 1) {
        // rotate the register arrays by one: the next weight moves into slot 0
        const float w0 = w[0];
        const float4 q0 = q[0];
        const float2 e0 = e[0];
        const bool l0 = loaded[0], d0 = dirty[0];
#pragma unroll
        for (int k = 0; k + 1 < UE_J; k++) {
          w[k] = w[k + 1];
          q[k] = q[k + 1];
          e[k] = e[k + 1];
          loaded[k] = loaded[k + 1];
          dirty[k] = dirty[k + 1];
        }
        w[UE_J - 1] = w0;
        q[UE_J - 1] = q0;
        e[UE_J - 1] = e0;
        loaded[UE_J - 1] = l0;
        dirty[UE_J - 1] = d0;
      }
    }
    __syncthreads();
  }
  if (i_ok) {
#pragma unroll
    for (int t = 0; t < UE_J; t++) {
      if (dirty[t]) {
        p.w[(long long)(j0 + t) * p.d_size + i] = w[t];
      }
    }
  }
}

template <int KIND, bool IMPLICIT, bool NOISY, int EJ, int UTJ>
static void launchUpdateVariant(const UpdateProblem &p, cudaStream_t stream) {
  constexpr int NT = UT_I * UTJ / EJ;
  static bool configured[64] = {};
  int dev = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    AB200_CUDA(cudaFuncSetAttribute(pulsedUpdateKernel<KIND, IMPLICIT, NOISY, EJ, UTJ>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)sizeof(UpdateSmem<NT, UTJ>)));
    configured[dev] = true;
  }
  dim3 grid((p.d_size + UT_I - 1) / UT_I, (p.x_size + UTJ - 1) / UTJ);
  AB200_CUDA(launchChained(pulsedUpdateKernel<KIND, IMPLICIT, NOISY, EJ, UTJ>, grid, dim3(NT),
                           sizeof(UpdateSmem<NT, UTJ>), stream, p));
}

template <int KIND, bool IMPLICIT, bool NOISY>
static void launchUpdateInstance(const UpdateProblem &p, dim3 grid, cudaStream_t stream) {
  // `grid` = CTAs of 64 d-lines x 16 x-lines. Four weights per thread (256 threads, four CTAs
  // per SM) once that grid fills the GPU several times over; one weight per thread (1024
  // threads) for small tiles; and CTAs of 64 x 4 weights (256 threads) when even that would
  // leave SMs without a CTA (a 256 x 256 tile is 64 CTAs of 64 x 16, but 256 of 64 x 4)
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    AB200_CUDA(cudaGetDevice(&dev));
    AB200_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  }
  const long long n = (long long)grid.x * grid.y;
  if (n >= 3LL * n_sm) {
    launchUpdateVariant<KIND, IMPLICIT, NOISY, 4, UT_J>(p, stream);
  } else if (n >= n_sm) {
    launchUpdateVariant<KIND, IMPLICIT, NOISY, 1, UT_J>(p, stream);
  } else {
    launchUpdateVariant<KIND, IMPLICIT, NOISY, 1, 4>(p, stream);
  }
}

// ---------------------------------------------------------------------------------------------
// Stochastic pulse trains: the update as a stream over the samples of one x-line.
//
// A warp owns 32 consecutive d-lines of ONE x-line. The x-line's pulse words are the same for all
// its lanes, so the walk over the samples is uniform across the warp: it visits the samples
// where the x word is not empty (a compacted list per x-line, built from the transposed x words
// and their bitmaps), loads the 32 d words of that sample with one coalesced access, and every
// lane counts its coincidences with AND + popc. No lane waits for another lane's candidates. The
// rare expensive part - applying the pulses - is decoupled: a lane queues its events (count,
// direction) and the warp applies the queued events together, so that most lanes have work in
// every round.
// ---------------------------------------------------------------------------------------------
constexpr int USP_POOL = 256; // Gaussians per warp pool (eight per lane and refill)

// xwT[line][sample] = xw[sample][line] for one 32 x 32 tile, plus the line's bitmap word of the
// non-empty samples
__global__ void __launch_bounds__(256)
    pulseTransposeKernel(const uint32_t *words, int n_lines, int m, int m_pad, uint32_t *wordsT,
                         uint32_t *nzT) {
  pdlEnter();
  __shared__ uint32_t tile[32][33];
  const int l0 = blockIdx.x * 32, s0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int s = s0 + r, l = l0 + threadIdx.x;
    tile[r][threadIdx.x] = (s < m && l < n_lines) ? words[(long long)s * n_lines + l] : 0u;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int l = l0 + r, sidx = s0 + threadIdx.x;
    const uint32_t w = tile[threadIdx.x][r];
    const uint32_t nz = __ballot_sync(0xffffffffu, w != 0u);
    if (l < n_lines) {
      wordsT[(long long)l * m_pad + sidx] = w;
      if (threadIdx.x == 0) {
        nzT[(long long)l * (m_pad / 32) + blockIdx.y] = nz;
      }
    }
  }
}

struct StreamUpdate {
  const uint32_t *xwT; // [x_size][m_pad]
  const uint32_t *xnzT; // [x_size][m_pad / 32]
  int m_pad;
  // compacted form of the same: per x-line the samples whose word is not empty, in order, and
  // their words with the sign bit flipped ([x_size][m_pad] each), and the number of entries before
  // every bitmap word ([x_size][m_pad / 32 + 1])
  const uint32_t *list_s, *list_x, *list_off;
};

// Compaction of the transposed x words of a line: the streaming kernel then reads (sample, word)
// pairs instead of walking a bitmap. One warp per line and segment of UCS_SEG_WORDS bitmap words;
// the warp first counts the entries of the line's earlier segments (a sum of popcounts over the
// bitmap, which stays in L2), then handles its bitmap words one at a time with the whole warp
// (lane = sample), so reads and writes are contiguous.
constexpr int UCS_SEG_WORDS = 128; // 4096 samples per warp

__global__ void __launch_bounds__(256)
    pulseCompactKernel(const uint32_t *wordsT, const uint32_t *nzT, int n_lines, int m_pad,
                       uint32_t *list_s, uint32_t *list_x, uint32_t *list_off) {
  pdlEnter();
  const int nw = m_pad >> 5;
  const int n_seg = (nw + UCS_SEG_WORDS - 1) / UCS_SEG_WORDS;
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)n_lines * n_seg) {
    return;
  }
  const int line = (int)(wid / n_seg), seg = (int)(wid - (long long)line * n_seg);
  const uint32_t *nz = nzT + (long long)line * nw;
  const uint32_t *xw = wordsT + (long long)line * m_pad;
  uint32_t *ls = list_s + (long long)line * m_pad, *lx = list_x + (long long)line * m_pad;
  uint32_t *off = list_off + (long long)line * (nw + 1);
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int w_begin = seg * UCS_SEG_WORDS;
  const int w_end = w_begin + UCS_SEG_WORDS < nw ? w_begin + UCS_SEG_WORDS : nw;
  // entries of this line before the segment
  uint32_t run = 0;
  for (int wd = lane; wd < w_begin; wd += 32) {
    run += (uint32_t)__popc(nz[wd]);
  }
  run = __reduce_add_sync(0xffffffffu, run);
  for (int w0 = w_begin; w0 < w_end; w0 += 32) {
    const int wd = w0 + lane;
    const uint32_t bits = wd < w_end ? nz[wd] : 0u;
    const uint32_t c = (uint32_t)__popc(bits);
    uint32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) {
        incl += v;
      }
    }
    const uint32_t excl = run + incl - c;
    if (wd < w_end) {
      off[wd] = excl;
    }
    const int nj = w_end - w0 < 32 ? w_end - w0 : 32;
    for (int j = 0; j < nj; j++) {
      const uint32_t bj = __shfl_sync(0xffffffffu, bits, j);
      if (bj == 0u) {
        continue;
      }
      const uint32_t basej = __shfl_sync(0xffffffffu, excl, j);
      const int smp = (w0 + j) * 32 + lane;
      const uint32_t xv = xw[smp];
      if ((bj >> lane) & 1u) {
        const uint32_t pos = basej + (uint32_t)__popc(bj & lt_mask);
        ls[pos] = (uint32_t)smp;
        lx[pos] = xv ^ 1u; // (x ^ d) & 1 is then the direction bit of an event
      }
    }
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0 && w_end == nw) {
    off[nw] = run;
  }
}

// The update itself: per walked sample two shuffles (sample, x word), the d word, AND, and - for
// the lanes with coincidences - one byte (count, direction) pushed into the lane's column of a
// queue in shared memory. The queues are drained together when one is nearly full, oldest event
// first: one pulse at a time with the clip after each, as in rpu_weight_updater.cpp:243-291. The
// Gaussians of the device noise come from a pool per warp in shared memory that all lanes refill
// together and take from without gaps (ballot + prefix count).
constexpr int USL_QCAP = 24; // events per lane between two drains

template <int KIND, bool NOISY>
__global__ void __launch_bounds__(256) pulsedUpdateListKernel(UpdateProblem p, StreamUpdate st) {
  pdlEnter();
  __shared__ float pool[8][USP_POOL];
  // rows padded by one word: lanes at different fill levels then fall into different banks
  __shared__ uint8_t evq[USL_QCAP][256 + 4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_dblk = (p.d_size + 31) >> 5;
  const long long task = (long long)blockIdx.x * 8 + warp;
  if (task >= (long long)n_dblk * p.x_size) {
    return;
  }
  const int j = (int)(task / n_dblk);
  const int i = (int)(task - (long long)j * n_dblk) * 32 + lane;
  const bool i_ok = i < p.d_size;
  const long long idx = (long long)j * p.d_size + (i_ok ? i : 0);
  float w = 0.0f;
  float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
  float2 e = make_float2(0.f, 0.f);
  if (i_ok) {
    w = p.w[idx];
    q = p.par4[idx];
    if (KIND != AB200_DEVICE_CONSTANT_STEP && KIND != AB200_DEVICE_EXP_STEP &&
        KIND != AB200_DEVICE_PIECEWISE_STEP) {
      e = p.par2[idx];
    }
  }
  const float w_in = w;
  const float std = p.dw_min_std;
  // chopped transfer compound: direction flipped when exactly one of the two lines is chopped
  uint32_t chop_flip = 0u;
  if (p.chop_x != nullptr) {
    chop_flip = (p.chop_x[j] != 0 ? 1u : 0u) ^ ((i_ok && p.chop_d[i] != 0) ? 1u : 0u);
  }
  int cnt = 0;
  int pool_pos = USP_POOL; // empty
  uint32_t refills = 0;
  const uint32_t lt_mask = (1u << lane) - 1u;

  auto drain = [&]() {
    const int rounds = __reduce_max_sync(0xffffffffu, cnt);
    for (int r = 0; r < rounds; r++) {
      int n = 0;
      bool down = false;
      if (r < cnt) {
        const uint32_t ev = evq[r][threadIdx.x];
        n = (int)(ev >> 1);
        down = (ev & 1u) != 0u;
      }
      for (int k = 0; __any_sync(0xffffffffu, k < n); k++) {
        const bool act = k < n;
        float xi = 0.0f;
        if (NOISY) {
          const uint32_t takers = __ballot_sync(0xffffffffu, act);
          if (pool_pos + __popc(takers) > USP_POOL) {
            // all lanes refill together; what is left of the old pool is dropped
            float z[8];
            gauss8(p.key, (uint64_t)(task * 32 + lane) | ((uint64_t)refills << 40), p.call, TAG_DEVICE, z);
            __syncwarp();
#pragma unroll
            for (int rr = 0; rr < 8; rr++) {
              pool[warp][rr * 32 + lane] = z[rr];
            }
            __syncwarp();
            refills++;
            pool_pos = 0;
          }
          if (act) {
            xi = std * pool[warp][pool_pos + __popc(takers & lt_mask)];
          }
          pool_pos += __popc(takers);
        }
        if (act) {
          w = pulseOnce<KIND>(w, down, q, e, xi, p.mult_noise, p.es0, p.es1, p.pw, p.pw_n);
        }
      }
    }
    cnt = 0;
  };

  const int nw = st.m_pad >> 5;
  const uint32_t *off = st.list_off + (long long)j * (nw + 1);
  const uint32_t *nz_line = st.xnzT + (long long)j * nw;
  const uint32_t *ls = st.list_s + (long long)j * st.m_pad;
  const uint32_t *lx = st.list_x + (long long)j * st.m_pad;
  // entries of the samples in [s_begin, s_end)
  auto entriesBefore = [&](int smp) -> uint32_t {
    const int wd = smp >> 5;
    if (wd >= nw) {
      return off[nw];
    }
    return off[wd] + (uint32_t)__popc(nz_line[wd] & ((1u << (smp & 31)) - 1u));
  };
  const uint32_t k_begin = entriesBefore(p.s_begin), k_end = entriesBefore(p.s_end);
  for (uint32_t k = k_begin; k < k_end; k += 32) {
    const uint32_t kk = k + lane;
    const uint32_t my_s = kk < k_end ? ls[kk] : 0u;
    const uint32_t my_x = kk < k_end ? lx[kk] : 0u;
    const int n_in = (int)(k_end - k < 32u ? k_end - k : 32u);
    for (int t = 0; t < n_in; t += 4) {
      // four samples at a time, so that their d words are in flight together
      uint32_t sv[4], xv[4], dwv[4];
#pragma unroll
      for (int c = 0; c < 4; c++) {
        sv[c] = __shfl_sync(0xffffffffu, my_s, (t + c) & 31);
        xv[c] = __shfl_sync(0xffffffffu, my_x, (t + c) & 31);
      }
#pragma unroll
      for (int c = 0; c < 4; c++) {
        dwv[c] = (t + c < n_in && i_ok) ? p.dw[(long long)sv[c] * p.d_size + i] : 0u;
      }
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const uint32_t both = xv[c] & dwv[c] & ~1u;
        if (both != 0u) {
          // equal line signs = decrease (rpu_weight_updater.cpp:246-268); the x sign is stored flipped
          evq[cnt][threadIdx.x] =
              (uint8_t)(((uint32_t)__popc(both) << 1) | (((xv[c] ^ dwv[c]) & 1u) ^ chop_flip));
          cnt++;
        }
      }
      if (__any_sync(0xffffffffu, cnt > USL_QCAP - 4)) {
        drain();
      }
    }
  }
  drain();
  if (i_ok && w != w_in) {
    p.w[idx] = w;
  }
}

template <int KIND>
static void launchStreamKind(const UpdateProblem &p, const StreamUpdate &st, cudaStream_t stream) {
  const long long tasks = (long long)((p.d_size + 31) / 32) * p.x_size;
  const unsigned blocks = (unsigned)((tasks + 7) / 8);
  if (p.dw_min_std > 0.0f) {
    AB200_CUDA(launchChained(pulsedUpdateListKernel<KIND, true>, dim3(blocks), dim3(256), 0, stream, p, st));
  } else {
    AB200_CUDA(launchChained(pulsedUpdateListKernel<KIND, false>, dim3(blocks), dim3(256), 0, stream, p, st));
  }
}

// the same problem in rows of pulse words: a sample has nseg of them
static UpdateProblem inRows(const UpdateProblem &p0) {
  UpdateProblem p = p0;
  const int nseg = p0.nseg > 0 ? p0.nseg : 1;
  p.m = p0.m * nseg;
  p.s_begin = p0.s_begin * nseg;
  p.s_end = p0.s_end * nseg;
  p.nseg = 1;
  return p;
}

static int g_update_path = 0;
void setUpdatePath(int mode) { g_update_path = mode; }

bool streamUpdateEligible(const UpdateProblem &p) {
  if (g_update_path == 1 || p.up.pulse_type != AB200_PULSE_STOCHASTIC_COMPRESSED) {
    return false;
  }
  return g_update_path == 2 || p.m * (p.nseg > 0 ? p.nseg : 1) >= kStreamUpdateMinBatch;
}

void launchPulseTranspose(const UpdateProblem &p0, uint32_t *xwT, uint32_t *xnzT, int m_pad,
                          cudaStream_t stream) {
  const UpdateProblem p = inRows(p0);
  dim3 grid((p.x_size + 31) / 32, m_pad / 32), block(32, 8);
  AB200_CUDA(launchChained(pulseTransposeKernel, grid, block, 0, stream, p.xw, p.x_size, p.m, m_pad, xwT,
                           xnzT));
  AB200_LAUNCH_CHECK();
}

void launchPulseCompact(const UpdateProblem &p0, const uint32_t *xwT, const uint32_t *xnzT, int m_pad,
                        uint32_t *list_s, uint32_t *list_x, uint32_t *list_off, cudaStream_t stream) {
  const UpdateProblem p = inRows(p0);
  const int n_seg = (m_pad / 32 + UCS_SEG_WORDS - 1) / UCS_SEG_WORDS;
  const unsigned blocks = (unsigned)(((long long)p.x_size * n_seg * 32 + 255) / 256);
  AB200_CUDA(launchChained(pulseCompactKernel, dim3(blocks), dim3(256), 0, stream, xwT, xnzT, p.x_size, m_pad,
                           list_s, list_x, list_off));
  AB200_LAUNCH_CHECK();
}

void launchPulsedUpdateStream(const UpdateProblem &p0, const uint32_t *xwT, const uint32_t *xnzT,
                              int m_pad, cudaStream_t stream, const uint32_t *list_s,
                              const uint32_t *list_x, const uint32_t *list_off) {
  const UpdateProblem p = inRows(p0);
  if (p.s_end <= p.s_begin) {
    return;
  }
  StreamUpdate st{xwT, xnzT, m_pad, list_s, list_x, list_off};
  switch (p.kind) {
  case AB200_DEVICE_CONSTANT_STEP:
    launchStreamKind<AB200_DEVICE_CONSTANT_STEP>(p, st, stream);
    break;
  case AB200_DEVICE_LINEAR_STEP:
  case AB200_DEVICE_SOFT_BOUNDS:
    launchStreamKind<AB200_DEVICE_LINEAR_STEP>(p, st, stream);
    break;
  case AB200_DEVICE_SOFT_BOUNDS_REFERENCE:
    launchStreamKind<AB200_DEVICE_SOFT_BOUNDS_REFERENCE>(p, st, stream);
    break;
  case AB200_DEVICE_POW_STEP:
    launchStreamKind<AB200_DEVICE_POW_STEP>(p, st, stream);
    break;
  case AB200_DEVICE_EXP_STEP:
    launchStreamKind<AB200_DEVICE_EXP_STEP>(p, st, stream);
    break;
  case AB200_DEVICE_PIECEWISE_STEP:
    launchStreamKind<AB200_DEVICE_PIECEWISE_STEP>(p, st, stream);
    break;
  default:
    AB200_FATAL("pulsed update: device kind not implemented");
  }
  AB200_LAUNCH_CHECK();
}

void launchPulsePrepare(const UpdateProblem &p, cudaStream_t stream) {
  if (p.m <= 0) {
    return;
  }
  AB200_CUDA(launchChained(pulsePrepareKernel, dim3(p.m), dim3(256), 0, stream, p));
  AB200_LAUNCH_CHECK();
}

void launchPulsedUpdate(const UpdateProblem &p0, cudaStream_t stream) {
  const UpdateProblem p = inRows(p0);
  if (p.s_end <= p.s_begin) {
    return;
  }
  dim3 grid((p.d_size + UT_I - 1) / UT_I, (p.x_size + UT_J - 1) / UT_J);
  const bool implicit = p.up.pulse_type == AB200_PULSE_DETERMINISTIC_IMPLICIT ||
                        p.up.pulse_type == AB200_PULSE_MEAN_COUNT;
  const bool noisy = p.dw_min_std > 0.0f;
#define AB200_UPD2(KIND, IMPL)                                                                     \
  if (noisy) {                                                                                     \
    launchUpdateInstance<KIND, IMPL, true>(p, grid, stream);                                       \
  } else {                                                                                         \
    launchUpdateInstance<KIND, IMPL, false>(p, grid, stream);                                      \
  }
#define AB200_UPD(KIND)                                                                            \
  if (implicit) {                                                                                  \
    AB200_UPD2(KIND, true)                                                                         \
  } else {                                                                                         \
    AB200_UPD2(KIND, false)                                                                        \
  }
  switch (p.kind) {
  case AB200_DEVICE_CONSTANT_STEP:
    AB200_UPD(AB200_DEVICE_CONSTANT_STEP);
    break;
  case AB200_DEVICE_LINEAR_STEP:
  case AB200_DEVICE_SOFT_BOUNDS:
    AB200_UPD(AB200_DEVICE_LINEAR_STEP);
    break;
  case AB200_DEVICE_SOFT_BOUNDS_REFERENCE:
    AB200_UPD(AB200_DEVICE_SOFT_BOUNDS_REFERENCE);
    break;
  case AB200_DEVICE_POW_STEP:
    AB200_UPD(AB200_DEVICE_POW_STEP);
    break;
  case AB200_DEVICE_EXP_STEP:
    AB200_UPD(AB200_DEVICE_EXP_STEP);
    break;
  case AB200_DEVICE_PIECEWISE_STEP:
    AB200_UPD(AB200_DEVICE_PIECEWISE_STEP);
    break;
  default:
    AB200_FATAL("pulsed update: device kind not implemented");
  }
#undef AB200_UPD
#undef AB200_UPD2
  AB200_LAUNCH_CHECK();
}

// Signed coincidence counts of sample 0 as int32 [d][x] (DenseBitLineMaker::makeCoincidences).
__global__ void coincidenceKernel(UpdateProblem p, int32_t *counts) {
  long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= (long long)p.x_size * p.d_size) {
    return;
  }
  int i = (int)(t / p.x_size), j = (int)(t % p.x_size);
  uint32_t xwv = p.xw[j], dwv = p.dw[i];
  int n;
  if (p.up.pulse_type == AB200_PULSE_DETERMINISTIC_IMPLICIT ||
      p.up.pulse_type == AB200_PULSE_MEAN_COUNT) {
    n = dwv == 0u ? 0 : (int)rintf(__fmul_rn(__uint_as_float(dwv), __uint_as_float(xwv)));
  } else {
    n = 0;
    const int nseg = p.nseg > 0 ? p.nseg : 1;
    for (int g = 0; g < nseg; g++) {
      xwv = p.xw[(long long)g * p.x_size + j];
      dwv = p.dw[(long long)g * p.d_size + i];
      const int c = __popc((xwv & dwv) >> 1);
      n += ((xwv ^ dwv) & 1u) != 0u ? -c : c;
    }
  }
  counts[t] = n;
}

// Pulse counters (kernelPulseCounter, src/rpucuda/cuda/pwu_kernel.h:1523-1620): a pass of its
// own over the prepared pulse words, one thread per weight, before the update applies them.
__global__ void __launch_bounds__(256)
    pulseCounterKernel(UpdateProblem p, unsigned long long *up, unsigned long long *down) {
  pdlEnter();
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= (long long)p.x_size * p.d_size) {
    return;
  }
  const int j = (int)(t / p.d_size), i = (int)(t % p.d_size); // the weights' own order [x][d]
  const bool implicit = p.up.pulse_type == AB200_PULSE_DETERMINISTIC_IMPLICIT ||
                        p.up.pulse_type == AB200_PULSE_MEAN_COUNT;
  const int nseg = p.nseg > 0 ? p.nseg : 1;
  unsigned long long n_up = 0, n_down = 0;
  for (int s = p.s_begin; s < p.s_end; s++) {
    const uint32_t *xw = p.xw + (long long)s * nseg * p.x_size;
    const uint32_t *dw = p.dw + (long long)s * nseg * p.d_size;
    if (implicit) {
      const uint32_t dwv = dw[i];
      const int n = dwv == 0u ? 0 : (int)rintf(__fmul_rn(__uint_as_float(dwv), __uint_as_float(xw[j])));
      // a positive product lowers the weight (w -= lr d x)
      if (n > 0) {
        n_down += (unsigned)n;
      } else {
        n_up += (unsigned)(-n);
      }
    } else {
      for (int g = 0; g < nseg; g++) {
        const uint32_t xwv = xw[(long long)g * p.x_size + j], dwv = dw[(long long)g * p.d_size + i];
        const unsigned c = (unsigned)__popc((xwv & dwv) >> 1);
        if (((xwv ^ dwv) & 1u) == 0u) {
          n_down += c;
        } else {
          n_up += c;
        }
      }
    }
  }
  up[t] += n_up;
  down[t] += n_down;
}

void launchPulseCounter(const UpdateProblem &p, unsigned long long *up, unsigned long long *down,
                        cudaStream_t stream) {
  if (p.s_end <= p.s_begin) {
    return;
  }
  const long long n = (long long)p.x_size * p.d_size;
  AB200_CUDA(launchChained(pulseCounterKernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, p, up,
                           down));
  AB200_LAUNCH_CHECK();
}

void launchCoincidences(const UpdateProblem &p, int32_t *counts_dx, cudaStream_t stream) {
  long long n = (long long)p.x_size * p.d_size;
  coincidenceKernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p, counts_dx);
  AB200_LAUNCH_CHECK();
}

// Floating-point update W[x][d] -= lr * sum_s x[s][x] d[s][d] (RPUSimple::updateMatrix,
// src/rpucuda/rpu.cpp:700-745), used by ideal devices / PulseType::None.
// `overwrite`: the target receives -lr * sum alone (delta-weight mode: beta = 0, rpu.cpp:1509-1511)
// CLIP_EACH: PulseType::NoneWithDevice - the rank-one update of every sample is followed by the
// clip to the element's bounds (rpu_weight_updater.cpp:216-223), so the samples are applied to the
// weight one after the other instead of being summed first.
template <bool CLIP_EACH>
__global__ void __launch_bounds__(256) fpUpdateKernel(UpdateProblem p, float lr_signed, int overwrite) {
  pdlEnter();
  __shared__ float xs[16][16 + 1];
  __shared__ float ds[16][64 + 1];
  const int ti = threadIdx.x & 63, tj = threadIdx.x >> 6; // 64 d-lines x 4 groups of 4 x-lines
  const int i = blockIdx.x * 64 + ti;
  const int jb = blockIdx.y * 16;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float wv[4] = {0.f, 0.f, 0.f, 0.f}, hi[4], lo[4];
  if (CLIP_EACH) {
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int j = jb + tj * 4 + t;
      hi[t] = lo[t] = 0.0f;
      if (i < p.d_size && j < p.x_size) {
        const long long idx = (long long)j * p.d_size + i;
        wv[t] = p.w[idx];
        if (p.par4 != nullptr) {
          const float4 q = p.par4[idx];
          hi[t] = q.z;
          lo[t] = q.w;
        } else {
          // no bounds: the digital accumulator of a mixed-precision compound
          hi[t] = 3.4e38f;
          lo[t] = -3.4e38f;
        }
      }
    }
  }
  for (int s0 = 0; s0 < p.m; s0 += 16) {
    {
      int ss = threadIdx.x >> 4, jj = threadIdx.x & 15;
      int gs = s0 + ss, gj = jb + jj;
      float v = 0.0f;
      if (gs < p.m && gj < p.x_size) {
        v = gj < p.x_real ? p.x[(long long)gs * p.x_ss + (long long)gj * p.x_fs] : 1.0f;
      }
      xs[ss][jj] = v;
    }
    for (int t = threadIdx.x; t < 16 * 64; t += 256) {
      int ss = t >> 6, ii = t & 63;
      int gs = s0 + ss, gi = blockIdx.x * 64 + ii;
      ds[ss][ii] = (gs < p.m && gi < p.d_size) ? p.d[(long long)gs * p.d_ss + (long long)gi * p.d_fs] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int ss = 0; ss < 16; ss++) {
      float dv = ds[ss][ti];
#pragma unroll
      for (int t = 0; t < 4; t++) {
        if (CLIP_EACH) {
          wv[t] = __fsub_rn(wv[t], __fmul_rn(__fmul_rn(lr_signed, dv), xs[ss][tj * 4 + t]));
          wv[t] = fmaxf(fminf(wv[t], hi[t]), lo[t]);
        } else {
          acc[t] = fmaf(xs[ss][tj * 4 + t], dv, acc[t]);
        }
      }
    }
    __syncthreads();
  }
  if (i < p.d_size) {
#pragma unroll
    for (int t = 0; t < 4; t++) {
      int j = jb + tj * 4 + t;
      if (j < p.x_size) {
        long long idx = (long long)j * p.d_size + i;
        if (CLIP_EACH) {
          p.w[idx] = wv[t];
        } else {
          p.w[idx] = overwrite ? -lr_signed * acc[t] : p.w[idx] - lr_signed * acc[t];
        }
      }
    }
  }
}

void launchFPUpdate(const UpdateProblem &p, float lr_signed, cudaStream_t stream, bool overwrite,
                    bool clip_each) {
  dim3 grid((p.d_size + 63) / 64, (p.x_size + 15) / 16);
  if (clip_each) {
    AB200_CUDA(launchChained(fpUpdateKernel<true>, grid, dim3(256), 0, stream, p, lr_signed, 0));
  } else {
    AB200_CUDA(launchChained(fpUpdateKernel<false>, grid, dim3(256), 0, stream, p, lr_signed,
                             overwrite ? 1 : 0));
  }
  AB200_LAUNCH_CHECK();
}

// Mixed-precision compound (MixedPrecRPUDevice::doDirectVectorUpdate,
// rpu_mixedprec_device.cpp:196-345): x and d of every sample quantised to n bins of their abs-max,
// q = clip(rint(v / width + u - 0.5), +-half) * width with width = amax / half, half = n / 2.
__global__ void __launch_bounds__(256)
    mixedQuantizeKernel(const float *x, long long x_ss, long long x_fs, int x_real, const float *d,
                        long long d_ss, long long d_fs, int x_size, int d_size, int n_x_bins, int n_d_bins,
                        int sr_x, int sr_d, PhiloxKey key, uint32_t call, float *qx, float *qd) {
  pdlEnter();
  __shared__ float sh[8];
  const int s = blockIdx.x;
  const float *xr = x + (long long)s * x_ss, *dr = d + (long long)s * d_ss;
  float xm = 0.0f, dm = 0.0f;
  for (int j = threadIdx.x; j < x_size; j += blockDim.x) {
    xm = fmaxf(xm, fabsf(j < x_real ? xr[(long long)j * x_fs] : 1.0f));
  }
  for (int i = threadIdx.x; i < d_size; i += blockDim.x) {
    dm = fmaxf(dm, fabsf(dr[(long long)i * d_fs]));
  }
  xm = blockMax(xm, sh);
  dm = blockMax(dm, sh);
  const float half_x = (float)(n_x_bins / 2), half_d = (float)(n_d_bins / 2);
  float x_width = __fdiv_rn(xm, half_x), d_width = __fdiv_rn(dm, half_d);
  x_width = x_width == 0.0f ? 1.0f : x_width;
  d_width = d_width == 0.0f ? 1.0f : d_width;
  for (int l = threadIdx.x; l < x_size + d_size; l += blockDim.x) {
    const bool is_x = l < x_size;
    const int idx = is_x ? l : l - x_size;
    const float v = is_x ? (idx < x_real ? xr[(long long)idx * x_fs] : 1.0f) : dr[(long long)idx * d_fs];
    const float width = is_x ? x_width : d_width, half = is_x ? half_x : half_d;
    float st = 0.0f;
    if (is_x ? sr_x : sr_d) {
      uint32_t r[4];
      philox4x32<7>((uint32_t)idx, (uint32_t)s, call, is_x ? TAG_PULSE_X : TAG_PULSE_D, key, r);
      st = __fadd_rn(u01(r[0]), -0.5f);
    }
    float q = rintf(__fadd_rn(__fdiv_rn(v, width), st));
    // (a zero stays a zero also where a single bin makes the width infinite: the reference skips it)
    q = q == 0.0f ? 0.0f : __fmul_rn(fminf(fmaxf(q, -half), half), width);
    if (is_x) {
      qx[(long long)s * x_size + idx] = q;
    } else {
      qd[(long long)s * d_size + idx] = q;
    }
  }
}

// The whole multiples of the granularity in rows [row0, row0 + n_rows) (mod d_size) of chi leave
// it as pulse counts (forwardUpdate, rpu_mixedprec_device.cpp:148-190); also writes the one-hot
// d vectors of the rows. chi is [x][d] like the weights.
__global__ void __launch_bounds__(256)
    mixedTruncateKernel(float *chi, int x_size, int d_size, int row0, int n_rows, float gran, float *counts,
                        float *onehot) {
  pdlEnter();
  const int j = blockIdx.y;
  const int row = (row0 + j) % d_size;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < x_size) {
    const long long idx = (long long)t * d_size + row;
    const float value = chi[idx];
    const float dw = truncf(__fdiv_rn(value, gran));
    counts[(long long)j * x_size + t] = dw;
    chi[idx] = __fsub_rn(value, __fmul_rn(dw, gran));
  }
  if (t < d_size) {
    onehot[(long long)j * d_size + t] = t == row ? 1.0f : 0.0f;
  }
}

void launchMixedQuantize(const UpdateProblem &p, int n_x_bins, int n_d_bins, int sr_x, int sr_d, float *qx,
                         float *qd, cudaStream_t stream) {
  AB200_CUDA(launchChained(mixedQuantizeKernel, dim3(p.m), dim3(256), 0, stream, p.x, p.x_ss, p.x_fs, p.x_real,
                           p.d, p.d_ss, p.d_fs, p.x_size, p.d_size, n_x_bins, n_d_bins, sr_x, sr_d, p.key,
                           p.call, qx, qd));
  AB200_LAUNCH_CHECK();
}

void launchMixedTruncate(float *chi, int x_size, int d_size, int row0, int n_rows, float gran, float *counts,
                         float *onehot, cudaStream_t stream) {
  const int width = x_size > d_size ? x_size : d_size;
  AB200_CUDA(launchChained(mixedTruncateKernel, dim3((width + 255) / 256, n_rows), dim3(256), 0, stream, chi,
                           x_size, d_size, row0, n_rows, gran, counts, onehot));
  AB200_LAUNCH_CHECK();
}

// Tiki-Taka read of one column of the fast tile: forward of a one-hot vector through the transfer
// IO (noise and bound management off) with alpha = -1
// (TransferRPUDevice::readVector / readAndUpdate, rpu_transfer_device.cpp:410-470). Also writes
// the one-hot vector that the following pulsed write uses as its x input.
__global__ void transferReadKernel(const float *w_fast, int col, int d_size, IOEff io,
                                   PhiloxKey key, uint32_t call, float *x_onehot, int x_size,
                                   float *r_out, float alpha) {
  pdlEnter();
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < x_size) {
    x_onehot[t] = t == col ? 1.0f : 0.0f;
  }
  if (t >= d_size) {
    return;
  }
  float y;
  if (io.is_perfect) {
    y = w_fast[(long long)col * d_size + t] * (alpha * io.out_scale);
  } else {
    float v = prepareInput(io, 1.0f, 1.0f);
    float acc = __fmul_rn(w_fast[(long long)col * d_size + t], v);
    float sigma = outputSigma(io, fabsf(v));
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (sigma > 0.0f) {
      gauss4(key, (uint64_t)(t >> 2), call, TAG_TRANSFER_READ, z);
    }
    bool ex = false;
    y = finalizeOutput(io, acc, sigma, z[t & 3], ex);
    y = __fmul_rn(y, __fmul_rn(io.out_scale, alpha));
  }
  r_out[t] = y;
}

// Buffered transfer (Tiki-Taka v2), BufferedTransferRPUDevice::readAndUpdate
// (src/rpucuda/rpu_buffered_transfer_device.cpp:178-208): omega = H + read * |lr|;
// n = trunc(omega / granularity) limited to +-max_steps; H keeps omega * momentum (forget) or
// omega minus the transferred part; the slow tile is then pulsed with d = -n.
__global__ void transferBufferKernel(float *buffer_col, float *read_inout, int d_size, float lr_abs,
                                     float bg, float max_steps, float momentum, int forget_buffer) {
  pdlEnter();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= d_size) {
    return;
  }
  const float omega = __fadd_rn(buffer_col[t], __fmul_rn(read_inout[t], lr_abs));
  const float n = fmaxf(fminf(truncf(__fdiv_rn(omega, bg)), max_steps), -max_steps);
  float h = omega;
  if (n != 0.0f) {
    const float sub_momentum = 1.0f - fmaxf(fminf(momentum, 1.0f), 0.0f);
    h = forget_buffer ? __fmul_rn(omega, momentum)
                      : __fsub_rn(omega, __fmul_rn(__fmul_rn(sub_momentum, n), bg));
  }
  buffer_col[t] = h;
  read_inout[t] = -n;
}

__global__ void __launch_bounds__(256)
    transferChopBufferKernel(float *buffer_col, float *read_inout, int d_size, float lr_scale,
                             float max_steps, float momentum, int forget_buffer, int no_buffer,
                             unsigned char *chop_in, int col, const unsigned char *chop_out,
                             int flip_in) {
  pdlEnter();
  // one CTA: the in chopper of the column is read by all threads before thread 0 flips it
  const bool in_chop = chop_in[col] != 0;
  const float sub_momentum = 1.0f - fmaxf(fminf(momentum, 1.0f), 0.0f);
  for (int t = threadIdx.x; t < d_size; t += blockDim.x) {
    float omega = no_buffer ? 0.0f : buffer_col[t];
    const float val = __fmul_rn(read_inout[t], lr_scale);
    omega = __fadd_rn(omega, (in_chop != (chop_out[t] != 0)) ? -val : val);
    float n = 0.0f;
    if (fabsf(omega) >= 1.0f) {
      n = fmaxf(fminf(truncf(omega), max_steps), -max_steps);
      omega = forget_buffer ? __fmul_rn(omega, momentum) : __fsub_rn(omega, __fmul_rn(sub_momentum, n));
    }
    buffer_col[t] = omega;
    read_inout[t] = -n;
  }
  __syncthreads();
  if (threadIdx.x == 0 && flip_in) {
    chop_in[col] = in_chop ? 0 : 1;
  }
}

__global__ void __launch_bounds__(256)
    transferDynamicBufferKernel(float *buffer_col, float *mean_col, float *past_col, float *read_inout,
                                int d_size, float lr_scale, float max_steps, float momentum,
                                int forget_buffer, float buffer_cap, float sample_momentum,
                                int previously_switched, unsigned char *chop_in, int col,
                                const unsigned char *chop_out, int flip_in) {
  pdlEnter();
  // one CTA: the in chopper of the column is read by all threads before thread 0 flips it
  const bool in_chop = chop_in[col] != 0;
  const float keep = 1.0f - sample_momentum, forget = 1.0f - momentum;
  for (int t = threadIdx.x; t < d_size; t += blockDim.x) {
    const float val = read_inout[t];
    float omega = buffer_col[t];
    float mu_past = past_col[t];
    const float mean = mean_col[t];
    if (previously_switched) {
      // a new chopper phase: the mean of the phase that ended becomes the reference
      mu_past = mean;
      past_col[t] = mean;
    }
    float dw = __fsub_rn(val, mu_past);
    dw = (in_chop != (chop_out[t] != 0)) ? -dw : dw;
    omega = __fadd_rn(omega, __fmul_rn(dw, lr_scale));
    float n = 0.0f;
    if (fabsf(omega) >= 1.0f) {
      n = fmaxf(fminf(truncf(omega), max_steps), -max_steps);
      if (forget_buffer) {
        omega = __fmul_rn(omega, momentum);
      } else {
        omega = __fsub_rn(omega, __fmul_rn(forget, n));
        if (buffer_cap > 0.0f) {
          omega = fminf(fmaxf(omega, -buffer_cap), buffer_cap);
        }
      }
    }
    buffer_col[t] = omega;
    read_inout[t] = -n;
    mean_col[t] = __fadd_rn(__fmul_rn(mean, keep), __fmul_rn(val, sample_momentum));
  }
  __syncthreads();
  if (threadIdx.x == 0 && flip_in) {
    chop_in[col] = in_chop ? 0 : 1;
  }
}

__global__ void __launch_bounds__(256)
    flipChoppersKernel(unsigned char *chop, int n, float prob, PhiloxKey key, uint32_t call) {
  pdlEnter();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) {
    return;
  }
  uint32_t r[4];
  philox4x32<7>((uint32_t)t, 0u, call, TAG_TRANSFER_READ ^ 0x01000000u, key, r);
  if (u01(r[0]) < prob) {
    chop[t] = chop[t] ? 0 : 1;
  }
}

void launchTransferChopBuffer(float *buffer_col, float *read_inout, int d_size, float lr_scale,
                              float max_steps, float momentum, int forget_buffer, int no_buffer,
                              unsigned char *chop_in, int col, const unsigned char *chop_out,
                              int flip_in, cudaStream_t stream) {
  AB200_CUDA(launchChained(transferChopBufferKernel, dim3(1), dim3(256), 0, stream, buffer_col, read_inout,
                           d_size, lr_scale, max_steps, momentum, forget_buffer, no_buffer, chop_in, col,
                           chop_out, flip_in));
  AB200_LAUNCH_CHECK();
}

void launchTransferDynamicBuffer(float *buffer_col, float *mean_col, float *past_col,
                                 float *read_inout, int d_size, float lr_scale, float max_steps,
                                 float momentum, int forget_buffer, float buffer_cap,
                                 float sample_momentum, int previously_switched,
                                 unsigned char *chop_in, int col, const unsigned char *chop_out,
                                 int flip_in, cudaStream_t stream) {
  AB200_CUDA(launchChained(transferDynamicBufferKernel, dim3(1), dim3(256), 0, stream, buffer_col, mean_col,
                           past_col, read_inout, d_size, lr_scale, max_steps, momentum, forget_buffer,
                           buffer_cap, sample_momentum, previously_switched, chop_in, col, chop_out,
                           flip_in));
  AB200_LAUNCH_CHECK();
}

void launchFlipChoppers(unsigned char *chop, int n, float prob, PhiloxKey key, uint32_t call,
                        cudaStream_t stream) {
  AB200_CUDA(launchChained(flipChoppersKernel, dim3((n + 255) / 256), dim3(256), 0, stream, chop, n, prob, key,
                           call));
  AB200_LAUNCH_CHECK();
}

void launchTransferBuffer(float *buffer_col, float *read_inout, int d_size, float lr_abs,
                          float buffer_granularity, float max_steps, float momentum,
                          int forget_buffer, cudaStream_t stream) {
  AB200_CUDA(launchChained(transferBufferKernel, dim3((d_size + 255) / 256), dim3(256), 0, stream,
                           buffer_col, read_inout, d_size, lr_abs, buffer_granularity, max_steps,
                           momentum, forget_buffer));
  AB200_LAUNCH_CHECK();
}

void launchTransferRead(const float *w_fast, int col, int d_size, const IOEff &io, PhiloxKey key,
                        uint32_t call, float *x_onehot, int x_size, float *r_out, float alpha,
                        cudaStream_t stream) {
  int n = d_size > x_size ? d_size : x_size;
  AB200_CUDA(launchChained(transferReadKernel, dim3((n + 255) / 256), dim3(256), 0, stream, w_fast, col,
                           d_size, io, key, call, x_onehot, x_size, r_out, alpha));
  AB200_LAUNCH_CHECK();
}

// dst[c][r] = src[r][c]  (host [d][x] <-> device [x][d] conversions)
__global__ void transposeKernel(const float *src, float *dst, int rows, int cols) {
  __shared__ float tile[32][33];
  int c = blockIdx.x * 32 + threadIdx.x, r = blockIdx.y * 32 + threadIdx.y;
  for (int k = 0; k < 32; k += 8) {
    if (c < cols && r + k < rows) {
      tile[threadIdx.y + k][threadIdx.x] = src[(long long)(r + k) * cols + c];
    }
  }
  __syncthreads();
  int oc = blockIdx.y * 32 + threadIdx.x, orow = blockIdx.x * 32 + threadIdx.y;
  for (int k = 0; k < 32; k += 8) {
    if (oc < rows && orow + k < cols) {
      dst[(long long)(orow + k) * rows + oc] = tile[threadIdx.x][threadIdx.y + k];
    }
  }
}

void launchTransposeDX(const float *src, float *dst, int rows, int cols, cudaStream_t stream) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transposeKernel<<<grid, block, 0, stream>>>(src, dst, rows, cols);
  AB200_LAUNCH_CHECK();
}

// PulsedRPUDevice::onSetWeights: clip to the per-element bounds (rpu_pulsed_device.cpp:545-571).
__global__ void clipKernel(float *w, const float4 *par4, long long n) {
  pdlEnter();
  long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    float4 q = par4[t];
    w[t] = fmaxf(fminf(w[t], q.z), q.w);
  }
}

void launchClipToBounds(float *w, const float4 *par4, long long n, cudaStream_t stream) {
  AB200_CUDA(launchChained(clipKernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, w, par4, n));
  AB200_LAUNCH_CHECK();
}

// Throughput of the arithmetic a coincidence costs at the least - one AND, one population count,
// one add per pair of pulse words - with everything in registers and four independent chains per
// thread: the integer ceiling the update kernel's pair rate is reported against.
__global__ void __launch_bounds__(256) popcPeakKernel(uint32_t *sink, int iters) {
  uint32_t a0 = threadIdx.x * 2654435761u + 1u, a1 = a0 ^ 0x9E3779B9u, a2 = a0 + 0x7F4A7C15u,
           a3 = a1 * 3u;
  const uint32_t b = blockIdx.x * 40503u + 0x5bd1e995u;
  uint32_t c0 = 0, c1 = 0, c2 = 0, c3 = 0;
  for (int k = 0; k < iters; k++) {
#pragma unroll
    for (int u = 0; u < 8; u++) {
      c0 += __popc(a0 & (b + c3));
      c1 += __popc(a1 & (b + c0));
      c2 += __popc(a2 & (b + c1));
      c3 += __popc(a3 & (b + c2));
    }
  }
  if (c0 + c1 + c2 + c3 == 0xFFFFFFFFu) {
    sink[0] = c0; // never true in practice: keeps the loop alive
  }
}

double measurePopcPeak(cudaStream_t stream) {
  int dev = 0, n_sm = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  AB200_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  uint32_t *sink = nullptr;
  AB200_CUDA(cudaMalloc(&sink, sizeof(uint32_t)));
  cudaEvent_t e0, e1;
  AB200_CUDA(cudaEventCreate(&e0));
  AB200_CUDA(cudaEventCreate(&e1));
  const int iters = 4096, blocks = n_sm * 8;
  popcPeakKernel<<<blocks, 256, 0, stream>>>(sink, 64); // warm-up
  AB200_CUDA(cudaEventRecord(e0, stream));
  popcPeakKernel<<<blocks, 256, 0, stream>>>(sink, iters);
  AB200_CUDA(cudaEventRecord(e1, stream));
  AB200_CUDA(cudaEventSynchronize(e1));
  float ms = 0.0f;
  AB200_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(sink);
  AB200_LAUNCH_CHECK();
  const double pairs = (double)blocks * 256.0 * (double)iters * 32.0;
  return pairs / ((double)ms * 1e-3);
}

__global__ void __launch_bounds__(256)
    addBlockKernel(const float *src, long long src_ld, float *dst, long long dst_ld, int cols,
                   long long n) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    const long long r = t / cols, c = t - r * cols;
    dst[r * dst_ld + c] += src[r * src_ld + c];
  }
}

void launchAddBlock(const float *src, long long src_ld, float *dst, long long dst_ld, int rows,
                    int cols, cudaStream_t stream) {
  const long long n = (long long)rows * cols;
  if (n <= 0) {
    return;
  }
  addBlockKernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(src, src_ld, dst, dst_ld, cols, n);
  AB200_LAUNCH_CHECK();
}

} // namespace ab200
