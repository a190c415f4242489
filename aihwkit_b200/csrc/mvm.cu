// IO-managed matrix-vector batch, generic CUDA-core path.
//
// Handles any tile shape, any activation layout (strided) and every IO setting of the path. The
// tensor-core kernel (mvm_tc.cu) takes over for large aligned problems; both use the same
// per-element helpers below so their results agree element by element, noise included.
//
// Reference semantics restated here:
//   noise management      src/rpucuda/rpu_forward_backward_pass.cpp:113-178
//   prepareInput (DAC)    src/rpucuda/rpu_forward_backward_pass.cpp:571-604
//   weight noise          src/rpucuda/rpu_forward_backward_pass.cpp:326-352
//   finalizeOutput (ADC)  src/rpucuda/rpu_forward_backward_pass.cpp:673-719
//   bound management      src/rpucuda/rpu_forward_backward_pass.cpp:935-988
//   backward              src/rpucuda/rpu_forward_backward_pass.cpp:991-1027
#include "mvm_common.cuh"
#include "tile.h"

namespace ab200 {

// ---------------------------------------------------------------------------------------------
// Kernel 1: per-sample noise management. One warp per sample (sample-contiguous layouts) or one
// thread per sample (feature-major layouts), so that loads stay coalesced either way.
// ---------------------------------------------------------------------------------------------
// `mode` 0: everything in one pass; 1: only the abs-max of every sample, written to p.sval;
// 2: the noise-management value of every sample is given in p.sval (the running-average types,
// whose value depends on the samples before it: nmAverageKernel sits between modes 1 and 2).
template <bool WARP_PER_SAMPLE>
__global__ void __launch_bounds__(256) nmScaleKernel(MvmProblem p, int mode) {
  pdlEnter();
  const IOEff &io = p.io;
  if (blockIdx.x == 0 && threadIdx.x == 0 && !p.backward && p.bm_stats) {
    // counters of the bound-management re-run of this pass
    p.bm_stats[0] = 0;
    p.bm_stats[1] = 0;
  }
  int lane = threadIdx.x & 31;
  int s = WARP_PER_SAMPLE ? (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5)
                          : (int)(blockIdx.x * (long long)blockDim.x + threadIdx.x);
  if (s >= p.m) {
    return;
  }
  const float *row = p.in + (long long)s * p.in_ss;
  NmStats st;
  if (mode != 2 && (nmNeedsStats(io) || mode == 1)) {
    if (WARP_PER_SAMPLE) {
      for (int k = lane; k < p.in_size; k += 32) {
        st.add(k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f);
      }
      st.warpReduce();
    } else {
      for (int k = 0; k < p.in_size; k++) {
        st.add(k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f);
      }
    }
  }
  if (mode == 1) {
    if (!WARP_PER_SAMPLE || lane == 0) {
      p.sval[s] = st.amax;
    }
    return;
  }
  float sval = mode == 2 ? p.sval[s] : nmValue(io, st);
  float scale = inputScale(io, sval, /*reduction=*/1.0f, !p.backward);
  const ElemRng g{p.key, p.call, (p.backward ? TAG_BWD_IN : TAG_FWD_IN) + p.noise_id};
  float vn = 0.0f;
  if (!io.is_perfect && io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f &&
      scale != 0.0f) {
    float acc = 0.0f;
    if (WARP_PER_SAMPLE) {
      for (int k = lane; k < p.in_size; k += 32) {
        float v = prepareInput(io, k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f, scale, g,
                               (uint32_t)s, (uint32_t)k);
        acc = fmaf(v, v, acc);
      }
      for (int o = 16; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
      }
    } else {
      for (int k = 0; k < p.in_size; k++) {
        float v = prepareInput(io, k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f, scale, g,
                               (uint32_t)s, (uint32_t)k);
        acc = fmaf(v, v, acc);
      }
    }
    vn = sqrtf(acc);
  }
  if (!WARP_PER_SAMPLE || lane == 0) {
    p.scale[s] = scale;
    p.sval[s] = sval;
    p.factor[s] = outputFactor(io, p.alpha, sval, scale, p.backward);
    p.vnorm[s] = vn;
    p.flags[s] = 0;
  }
}

// AverageAbsMax / AverageAbsMaxSingleValue (rpu_forward_backward_pass.cpp:139-150): the value of
// sample s is the running value after sample s, s <- s (1 - decay) + decay * amax_s, started by
// the first sample the tile ever sees. A recurrence over the samples in their order: one thread.
__global__ void nmAverageKernel(float *sval, int m, float decay, float *state) {
  pdlEnter();
  if (blockIdx.x != 0 || threadIdx.x != 0) {
    return;
  }
  float a = *state;
  for (int s = 0; s < m; s++) {
    const float amax = sval[s];
    a = a < 0.0f ? amax : __fadd_rn(__fmul_rn(a, __fsub_rn(1.0f, decay)), __fmul_rn(decay, amax));
    sval[s] = a;
  }
  *state = a;
}

// ---------------------------------------------------------------------------------------------
// Kernel 2: tiled fp32 product with the DAC fused into the operand load and noise / ADC / clip /
// bound flag / rescale fused into the epilogue.
// ---------------------------------------------------------------------------------------------
// T x T outputs per thread, 16 x 16 threads: 64 x 64 outputs per CTA for large problems, 32 x 32 or
// 16 x 16 when the larger tile would leave most SMs without a CTA (a 256 x 256 tile with a batch of
// 64 is four CTAs of 64 x 64, but 64 of 16 x 16).
// The K step of a CTA grows as its tile shrinks: the small tiles serve small problems, whose time is
// the latency of the K loop (global load -> DAC -> shared memory -> barrier per step), not its
// arithmetic, so they take 64 or 32 features per step with several loads in flight per thread.

// PCM ("line chain"): also accumulate per output sum_k |w| v^2 (variance factor of the PCMRead
// weight noise), sum_k |w| |v| (line current) and sum_k w v posw(k) (position-weighted product) for
// the IR drop, and run the long output chain (lineChain) instead of the merged noise draw.
// NMF (small problems, T = 1): the noise management of the CTA's sixteen rows runs in the prologue
// instead of a kernel of its own - sixteen threads per row reduce the row's statistics, every
// column CTA of a row block repeats that (a few KB), and the first one leaves the per-row values
// for the bound-management re-run. One launch less per pass where launches are what a pass costs.
// PN (with PCM): the negative and the positive prepared inputs accumulate separately, with the
// norm of each half, and the epilogue runs the analog chain of the line once per half before it
// adds them in front of (pos_neg = 1) or behind (pos_neg = 2) the output stage
// (computeAnalogMV, rpu_forward_backward_pass.cpp:820-876).
template <bool A_K_FAST, bool B_N_FAST, int T, bool PCM, bool NMF = false, bool PN = false>
__global__ void __launch_bounds__(256) mvmSimtKernel(MvmProblem p) {
  static_assert(!PN || PCM, "separate passes use the line-chain variant");
  constexpr int S = PN ? 2 : 1; // accumulator sets: [negative inputs, positive inputs] or one
  pdlEnter();
  constexpr int BM = 16 * T, BN = 16 * T;
  constexpr int BK = T == 1 ? 64 : (T == 2 ? 32 : 16);
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  __shared__ float s_scale[BM];
  __shared__ float s_fac[NMF ? BM : 1];
  const IOEff &io = p.io;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const int K = p.in_size, N = p.out_size;
  const ElemRng g{p.key, p.call, (p.backward ? TAG_BWD_IN : TAG_FWD_IN) + p.noise_id};

  if (NMF) {
    // BM = 16 rows, 16 threads per row
    const int r = tid >> 4, part = tid & 15;
    const int gr = row0 + r;
    NmStats st;
    if (gr < p.m && nmNeedsStats(io)) {
      const float *row = p.in + (long long)gr * p.in_ss;
      for (int k = part; k < K; k += 16) {
        st.add(k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f);
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      st.amax = fmaxf(st.amax, __shfl_xor_sync(0xffffffffu, st.amax, o));
      st.vmax = fmaxf(st.vmax, __shfl_xor_sync(0xffffffffu, st.vmax, o));
      st.psum += __shfl_xor_sync(0xffffffffu, st.psum, o);
      st.nsum += __shfl_xor_sync(0xffffffffu, st.nsum, o);
    }
    if (part == 0) {
      float scale = 0.0f, fac = 0.0f;
      if (gr < p.m) {
        const float sval = nmValue(io, st);
        scale = inputScale(io, sval, /*reduction=*/1.0f, !p.backward);
        fac = outputFactor(io, p.alpha, sval, scale, p.backward);
        if (blockIdx.x == 0) {
          // what the bound-management re-run reads; the flags are zero between passes (the
          // re-run clears the ones it has served)
          p.scale[gr] = scale;
          p.sval[gr] = sval;
          p.factor[gr] = fac;
          p.vnorm[gr] = 0.0f;
        }
      }
      s_scale[r] = scale;
      s_fac[NMF ? r : 0] = fac;
    }
    if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0 && !p.backward && p.bm_stats) {
      p.bm_stats[0] = 0;
      p.bm_stats[1] = 0;
    }
  } else if (tid < BM) {
    int r = row0 + tid;
    s_scale[tid] = r < p.m ? p.scale[r] : 0.0f;
  }
  __syncthreads();

  float acc[S][T][T];
  float acc2[S][PCM ? T : 1][PCM ? T : 1], acc_c[S][PCM ? T : 1][PCM ? T : 1], acc_i[S][PCM ? T : 1][PCM ? T : 1];
  float vn2[S][PN ? T : 1]; // PN: squared norm of each half of the prepared input, per row
#pragma unroll
  for (int h = 0; h < S; h++) {
#pragma unroll
    for (int i = 0; i < T; i++) {
      vn2[h][PN ? i : 0] = 0.0f;
#pragma unroll
      for (int j = 0; j < T; j++) {
        acc[h][i][j] = 0.0f;
        if (PCM) {
          acc2[h][PCM ? i : 0][PCM ? j : 0] = 0.0f;
          acc_c[h][PCM ? i : 0][PCM ? j : 0] = 0.0f;
          acc_i[h][PCM ? i : 0][PCM ? j : 0] = 0.0f;
        }
      }
    }
  }

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = tid; e < BM * BK; e += 256) {
      int r, kk;
      if (A_K_FAST) {
        kk = e % BK;
        r = e / BK;
      } else {
        r = e % BM;
        kk = e / BM;
      }
      int gr = row0 + r, gk = k0 + kk;
      float v = 0.0f;
      if (gr < p.m && gk < K) {
        float sc = s_scale[r];
        if (sc != 0.0f) {
          float xin = gk < p.in_real ? p.in[(long long)gr * p.in_ss + (long long)gk * p.in_fs] : 1.0f;
          v = prepareInput(io, xin, sc, g, (uint32_t)gr, (uint32_t)gk);
        }
      }
      As[kk][r] = v;
    }
#pragma unroll
    for (int e = tid; e < BN * BK; e += 256) {
      int n, kk;
      if (B_N_FAST) {
        n = e % BN;
        kk = e / BN;
      } else {
        kk = e % BK;
        n = e / BK;
      }
      int gk = k0 + kk, gn = col0 + n;
      Bs[kk][n] = (gk < K && gn < N) ? p.w[(long long)gk * p.wk + (long long)gn * p.wn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[T], b[T];
      const float posw = PCM ? irPosWeight(k0 + kk, K) : 0.0f;
#pragma unroll
      for (int i = 0; i < T; i++) {
        a[i] = As[kk][ty * T + i];
      }
#pragma unroll
      for (int j = 0; j < T; j++) {
        b[j] = Bs[kk][tx * T + j];
      }
#pragma unroll
      for (int h = 0; h < S; h++) {
#pragma unroll
        for (int i = 0; i < T; i++) {
          // PN: half 0 takes the negative inputs, half 1 the positive ones
          const float ah = PN ? (h == 0 ? fminf(a[i], 0.0f) : fmaxf(a[i], 0.0f)) : a[i];
          if (PN) {
            vn2[h][PN ? i : 0] = fmaf(ah, ah, vn2[h][PN ? i : 0]);
          }
#pragma unroll
          for (int j = 0; j < T; j++) {
            acc[h][i][j] = fmaf(ah, b[j], acc[h][i][j]);
            if (PCM) {
              const float ab = fabsf(b[j]);
              acc2[h][PCM ? i : 0][PCM ? j : 0] = fmaf(ah * ah, ab, acc2[h][PCM ? i : 0][PCM ? j : 0]);
              acc_c[h][PCM ? i : 0][PCM ? j : 0] = fmaf(fabsf(ah), ab, acc_c[h][PCM ? i : 0][PCM ? j : 0]);
              acc_i[h][PCM ? i : 0][PCM ? j : 0] = fmaf(ah * posw, b[j], acc_i[h][PCM ? i : 0][PCM ? j : 0]);
            }
          }
        }
      }
    }
    __syncthreads();
  }

  // noise blocks of four columns, an even number per row (two blocks share one Philox call); a
  // thread with fewer than four columns draws its block and takes its columns from it
  const uint64_t n4 = (uint64_t)(((N + 7) >> 3) << 1);
  const uint32_t tag = (p.backward ? TAG_BWD_OUT : TAG_FWD_OUT) + p.noise_id;
  const uint32_t tag_u = (p.backward ? TAG_BWD_OUT_U : TAG_FWD_OUT_U) + p.noise_id;
#pragma unroll
  for (int i = 0; i < T; i++) {
    int r = row0 + ty * T + i;
    if (r >= p.m) {
      continue;
    }
    int c = col0 + tx * T;
    if (c >= N) {
      continue;
    }
    float sc = s_scale[ty * T + i];
    float fac = NMF ? s_fac[NMF ? ty * T + i : 0] : p.factor[r];
    float y[T];
#pragma unroll
    for (int j = 0; j < T; j++) {
      y[j] = acc[S - 1][i][j]; // PN: the positive half
    }
    bool exceeded = false;
    if (sc == 0.0f) {
#pragma unroll
      for (int j = 0; j < T; j++) {
        y[j] = 0.0f;
      }
    } else if (io.is_perfect) {
#pragma unroll
      for (int j = 0; j < T; j++) {
        y[j] *= fac;
      }
    } else {
      const bool line_sigma = p.out_noise_vals != nullptr;
      const float vn = NMF ? 0.0f : p.vnorm[r];
      float sigma = PCM ? io.out_noise : outputSigma(io, vn);
      const uint64_t blk = (uint64_t)r * n4 + (uint64_t)(c >> 2);
      const bool w_draw = PCM && io.w_noise > 0.0f && io.w_noise_type != AB200_WNOISE_NONE;
      float z[4] = {0.f, 0.f, 0.f, 0.f};
      if (sigma > 0.0f || line_sigma) {
        gauss4(p.key, blk, p.call, tag, z);
      }
      float zw[4] = {0.f, 0.f, 0.f, 0.f};
      if (w_draw) {
        // the weight noise enters before the non-linearity: a draw of its own
        gauss4(p.key, blk, p.call, tag ^ 0x04000000u, zw);
      }
      float u[4] = {0.5f, 0.5f, 0.5f, 0.5f};
      if (io.out_sto_round) {
        uniform4(p.key, blk, p.call, tag_u, u);
      }
      // PN: the draws of the pass over the negative inputs
      float zn[4] = {0.f, 0.f, 0.f, 0.f}, zwn[4] = {0.f, 0.f, 0.f, 0.f}, un[4] = {0.5f, 0.5f, 0.5f, 0.5f};
      if (PN) {
        if (io.pos_neg == 2 && (sigma > 0.0f || line_sigma)) {
          gauss4(p.key, blk, p.call, tag ^ 0x08000000u, zn);
        }
        if (w_draw) {
          gauss4(p.key, blk, p.call, tag ^ 0x0c000000u, zwn);
        }
        if (io.pos_neg == 2 && io.out_sto_round) {
          uniform4(p.key, blk, p.call, tag_u ^ 0x08000000u, un);
        }
      }
      const LineChain lc{p.v_offset, p.out_nl, p.nl_factor, __fdiv_rn((float)K, io.ir_g_ratio)};
#pragma unroll
      for (int j = 0; j < T; j++) {
        const int q = (c + j) & 3; // T divides 4 and c is a multiple of T: same block for all j
        float yn = 0.0f;
        if (c + j < N) {
          if (line_sigma) {
            sigma = PCM ? p.out_noise_vals[c + j] : outputSigmaLine(io, vn, p.out_noise_vals, c + j, 0.0f);
          }
          if (PCM) {
            y[j] = lineChain(io, lc, y[j], c + j, acc_c[S - 1][PCM ? i : 0][PCM ? j : 0],
                             acc_i[S - 1][PCM ? i : 0][PCM ? j : 0], acc2[S - 1][PCM ? i : 0][PCM ? j : 0],
                             PN ? sqrtf(vn2[S - 1][PN ? i : 0]) : vn, zw[q], /*with_nl=*/!PN);
          }
          if (PN) {
            yn = lineChain(io, lc, acc[0][i][j], c + j, acc_c[0][PCM ? i : 0][PCM ? j : 0],
                           acc_i[0][PCM ? i : 0][PCM ? j : 0], acc2[0][PCM ? i : 0][PCM ? j : 0],
                           sqrtf(vn2[0][PN ? i : 0]), zwn[q], /*with_nl=*/false);
            if (io.pos_neg == 2) {
              yn = lineNonLinearity(lc, yn, c + j);
              y[j] = lineNonLinearity(lc, y[j], c + j);
            } else {
              y[j] = lineNonLinearity(lc, __fadd_rn(y[j], yn), c + j); // analog sum, then the output stage
            }
          }
        }
        if (PN && io.pos_neg == 2) {
          // each pass through its own output stage, digital sum
          yn = finalizeOutput(io, yn, sigma, zn[q], exceeded, un[q]);
          y[j] = finalizeOutput(io, y[j], sigma, z[q], exceeded, u[q]);
          y[j] = __fadd_rn(y[j], yn) * fac;
        } else {
          y[j] = finalizeOutput(io, y[j], sigma, z[q], exceeded, u[q]) * fac;
        }
      }
    }
    if (exceeded && io.bm != AB200_BM_NONE) {
      atomicOr(&p.flags[r], 1);
    }
#pragma unroll
    for (int j = 0; j < T; j++) {
      if (c + j < p.out_store) {
        float *o = mvmOutPtr(p, r, c + j);
        *o = p.accumulate ? *o + y[j] : y[j];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Kernel 3: iterative bound management. Only samples whose first round clipped are re-run; each
// is an independent mat-vec with a halved input scale per round, exactly the per-sample loop of
// the reference CPU tile. Nothing is copied to the host.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bmRerunKernel(MvmProblem p) {
  pdlEnter();
  extern __shared__ float v_sh[]; // K prepared inputs
  const IOEff &io = p.io;
  const int K = p.in_size, N = p.out_size;
  const uint64_t n4 = (uint64_t)(((N + 7) >> 3) << 1);
  for (int r = blockIdx.x; r < p.m; r += gridDim.x) {
    if (p.flags[r] == 0) {
      continue;
    }
    float sval = p.sval[r];
    const float *row = p.in + (long long)r * p.in_ss;
    const bool gathered = p.gather.idx != nullptr; // rows read through an index array
    float reduction = 1.0f;
    float scale = 1.0f;
    int round = 0;
    bool done = false;
    while (!done) {
      reduction *= 2.0f;
      round++;
      if (round == 1 && io.bm == AB200_BM_ITERATIVE_WORST_CASE && io.nm != AB200_NM_ABS_MAX_NP_SUM) {
        // IterativeWorstCase: the first re-run switches to the AbsMaxNPSum scale and starts the
        // halving again from there (rpu_forward_backward_pass.cpp:945-950)
        NmStats st;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
          st.add(gathered ? gatherRowElement(p.gather, p.in, r, k)
                          : (k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f));
        }
        st.warpReduce();
        __shared__ float st_sh[8][3];
        if ((threadIdx.x & 31) == 0) {
          st_sh[threadIdx.x >> 5][0] = st.amax;
          st_sh[threadIdx.x >> 5][1] = st.psum;
          st_sh[threadIdx.x >> 5][2] = st.nsum;
        }
        __syncthreads();
        NmStats all;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) {
          all.amax = fmaxf(all.amax, st_sh[i][0]);
          all.psum += st_sh[i][1];
          all.nsum += st_sh[i][2];
        }
        __syncthreads();
        sval = nmValueNPSum(io, all);
        reduction = 1.0f;
      }
      scale = inputScale(io, sval, reduction, true);
      const ElemRng g{p.key, p.call, TAG_FWD_IN + p.noise_id + (uint32_t)round * 0x10000u};
      // squared norm of the prepared input, negative and positive half apart (the separate
      // passes of pos_neg each see their own half)
      float nacc_n = 0.0f, nacc_p = 0.0f;
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float xin = gathered ? gatherRowElement(p.gather, p.in, r, k)
                                   : (k < p.in_real ? row[(long long)k * p.in_fs] : 1.0f);
        float v = prepareInput(io, xin, scale, g, (uint32_t)r, (uint32_t)k);
        v_sh[k] = v;
        if (v < 0.0f) {
          nacc_n = fmaf(v, v, nacc_n);
        } else {
          nacc_p = fmaf(v, v, nacc_p);
        }
      }
      float vn = 0.0f, vn_n = 0.0f, vn_p = 0.0f;
      if (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f) {
        for (int o = 16; o > 0; o >>= 1) {
          nacc_n += __shfl_xor_sync(0xffffffffu, nacc_n, o);
          nacc_p += __shfl_xor_sync(0xffffffffu, nacc_p, o);
        }
        __shared__ float red2_sh[8][2];
        if ((threadIdx.x & 31) == 0) {
          red2_sh[threadIdx.x >> 5][0] = nacc_n;
          red2_sh[threadIdx.x >> 5][1] = nacc_p;
        }
        __syncthreads();
        float tn = 0.0f, tp = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) {
          tn += red2_sh[i][0];
          tp += red2_sh[i][1];
        }
        vn = sqrtf(tn + tp);
        vn_n = sqrtf(tn);
        vn_p = sqrtf(tp);
      }
      __syncthreads();
      const bool pcm = ioNeedsLineChain(io);
      const int pos_neg = io.pos_neg;
      float sigma = pcm ? io.out_noise : outputSigma(io, vn);
      const bool line_sigma = p.out_noise_vals != nullptr;
      const LineChain lc{p.v_offset, p.out_nl, p.nl_factor, __fdiv_rn((float)K, io.ir_g_ratio)};
      const uint32_t round_tag = TAG_FWD_OUT + p.noise_id + (uint32_t)round * 0x10000u;
      const uint32_t round_tag_u = TAG_FWD_OUT_U + p.noise_id + (uint32_t)round * 0x10000u;
      const bool w_draw = io.w_noise > 0.0f && io.w_noise_type != AB200_WNOISE_NONE;
      int fail = 0;
      for (int n = threadIdx.x; n < N; n += blockDim.x) {
        // accumulator sets: [0] the only pass, or the pass over the positive inputs; [1] the
        // pass over the negative inputs
        float acc[2] = {0.0f, 0.0f}, acc2[2] = {0.0f, 0.0f}, acc_c[2] = {0.0f, 0.0f}, acc_i[2] = {0.0f, 0.0f};
        const float *wp = p.w + (long long)n * p.wn;
        if (pos_neg != 0) {
          for (int k = 0; k < K; k++) {
            const float wv = wp[(long long)k * p.wk], v = v_sh[k];
            const float vp = fmaxf(v, 0.0f), vm = fminf(v, 0.0f), pw = irPosWeight(k, K), aw = fabsf(wv);
            acc[0] = fmaf(vp, wv, acc[0]);
            acc2[0] = fmaf(vp * vp, aw, acc2[0]);
            acc_c[0] = fmaf(vp, aw, acc_c[0]);
            acc_i[0] = fmaf(vp * pw, wv, acc_i[0]);
            acc[1] = fmaf(vm, wv, acc[1]);
            acc2[1] = fmaf(vm * vm, aw, acc2[1]);
            acc_c[1] = fmaf(-vm, aw, acc_c[1]);
            acc_i[1] = fmaf(vm * pw, wv, acc_i[1]);
          }
        } else if (pcm) {
          for (int k = 0; k < K; k++) {
            const float wv = wp[(long long)k * p.wk], v = v_sh[k];
            acc[0] = fmaf(v, wv, acc[0]);
            acc2[0] = fmaf(v * v, fabsf(wv), acc2[0]);
            acc_c[0] = fmaf(fabsf(v), fabsf(wv), acc_c[0]);
            acc_i[0] = fmaf(v * irPosWeight(k, K), wv, acc_i[0]);
          }
        } else {
          for (int k = 0; k < K; k++) {
            acc[0] = fmaf(v_sh[k], wp[(long long)k * p.wk], acc[0]);
          }
        }
        if (line_sigma) {
          sigma = pcm ? p.out_noise_vals[n] : outputSigmaLine(io, vn, p.out_noise_vals, n, 0.0f);
        }
        const uint64_t blk = (uint64_t)r * n4 + (uint64_t)(n >> 2);
        if (pcm) {
          float zw[4] = {0.f, 0.f, 0.f, 0.f};
          if (w_draw) {
            gauss4(p.key, blk, p.call, round_tag ^ 0x04000000u, zw);
          }
          acc[0] = lineChain(io, lc, acc[0], n, acc_c[0], acc_i[0], acc2[0], pos_neg != 0 ? vn_p : vn, zw[n & 3],
                             /*with_nl=*/pos_neg == 0);
          if (pos_neg != 0) {
            float zwn[4] = {0.f, 0.f, 0.f, 0.f};
            if (w_draw) {
              gauss4(p.key, blk, p.call, round_tag ^ 0x0c000000u, zwn);
            }
            acc[1] = lineChain(io, lc, acc[1], n, acc_c[1], acc_i[1], acc2[1], vn_n, zwn[n & 3], /*with_nl=*/false);
            if (pos_neg == 2) {
              acc[0] = lineNonLinearity(lc, acc[0], n);
              acc[1] = lineNonLinearity(lc, acc[1], n);
            } else {
              acc[0] = lineNonLinearity(lc, __fadd_rn(acc[0], acc[1]), n); // analog sum, then the output stage
            }
          }
        }
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        if (sigma > 0.0f) {
          gauss4(p.key, blk, p.call, round_tag, z);
        }
        float u[4] = {0.5f, 0.5f, 0.5f, 0.5f};
        if (io.out_sto_round) {
          uniform4(p.key, blk, p.call, round_tag_u, u);
        }
        bool ex = false;
        float y;
        if (pos_neg == 2) {
          float zn[4] = {0.f, 0.f, 0.f, 0.f}, un[4] = {0.5f, 0.5f, 0.5f, 0.5f};
          if (sigma > 0.0f) {
            gauss4(p.key, blk, p.call, round_tag ^ 0x08000000u, zn);
          }
          if (io.out_sto_round) {
            uniform4(p.key, blk, p.call, round_tag_u ^ 0x08000000u, un);
          }
          const float yn = finalizeOutput(io, acc[1], sigma, zn[n & 3], ex, un[n & 3]);
          y = __fadd_rn(finalizeOutput(io, acc[0], sigma, z[n & 3], ex, u[n & 3]), yn);
        } else {
          y = finalizeOutput(io, acc[0], sigma, z[n & 3], ex, u[n & 3]);
        }
        fail |= ex ? 1 : 0;
        if (n < p.out_store) {
          *mvmOutPtr(p, r, n) = y;
        }
      }
      int any_fail = __syncthreads_or(fail);
      done = !any_fail || ((int)reduction > io.max_bm_factor) ||
             (io.res_in > 0.0f && reduction > __fdiv_rn(io.max_bm_res, io.res_in));
    }
    float fac = outputFactor(io, p.alpha, sval, scale, false);
    for (int n = threadIdx.x; n < N && n < p.out_store; n += blockDim.x) {
      *mvmOutPtr(p, r, n) *= fac;
    }
    if (threadIdx.x == 0) {
      atomicAdd(&p.bm_stats[0], 1);
      atomicMax(&p.bm_stats[1], __float_as_int(reduction));
      p.flags[r] = 0; // served: the flags are zero again when the next pass starts
    }
    __syncthreads();
  }
}

void launchMvmSimt(const MvmProblem &p, cudaStream_t stream) {
  // noise management
  bool sample_contig = p.in_fs == 1;
  auto nmPass = [&](int mode) {
    if (sample_contig) {
      int blocks = (int)(((long long)p.m * 32 + 255) / 256);
      AB200_CUDA(launchChained(nmScaleKernel<true>, dim3(blocks), dim3(256), 0, stream, p, mode));
    } else {
      AB200_CUDA(launchChained(nmScaleKernel<false>, dim3((p.m + 255) / 256), dim3(256), 0, stream, p, mode));
    }
    AB200_LAUNCH_CHECK();
  };
  const bool running = !p.io.is_perfect && (p.io.nm == AB200_NM_AVERAGE_ABS_MAX ||
                                            p.io.nm == AB200_NM_AVERAGE_ABS_MAX_SINGLE_VALUE);
  // small problems (the 16 x 16 tile is chosen below) without per-row norms or running values:
  // the noise management goes into the prologue of the product kernel
  static int n_sm = 0; // SMs of the GPUs of this process (one kind per process)
  if (n_sm == 0) {
    int dev = 0;
    AB200_CUDA(cudaGetDevice(&dev));
    AB200_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  }
  const long long ctas2 = (long long)((p.out_size + 31) / 32) * ((p.m + 31) / 32);
  const bool fused_nm = !running && !ioNeedsLineChain(p.io) && ctas2 < n_sm && p.in_size <= 4096 &&
                        !(p.io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && p.io.w_noise > 0.0f &&
                          !p.io.is_perfect);
  if (fused_nm) {
    dim3 grid((p.out_size + 15) / 16, (p.m + 15) / 16);
    const bool a_k = p.in_fs == 1, b_n = p.wn == 1;
    if (a_k && b_n) {
      AB200_CUDA(launchChained(mvmSimtKernel<true, true, 1, false, true>, grid, dim3(256), 0, stream, p));
    } else if (a_k) {
      AB200_CUDA(launchChained(mvmSimtKernel<true, false, 1, false, true>, grid, dim3(256), 0, stream, p));
    } else if (b_n) {
      AB200_CUDA(launchChained(mvmSimtKernel<false, true, 1, false, true>, grid, dim3(256), 0, stream, p));
    } else {
      AB200_CUDA(launchChained(mvmSimtKernel<false, false, 1, false, true>, grid, dim3(256), 0, stream, p));
    }
    AB200_LAUNCH_CHECK();
    return;
  }
  if (running) {
    if (!p.nm_state) {
      AB200_FATAL("running-average noise management needs a tile (its state lives there)");
    }
    nmPass(1);
    AB200_CUDA(launchChained(nmAverageKernel, dim3(1), dim3(32), 0, stream, p.sval, p.m, p.io.nm_decay,
                             p.nm_state));
    AB200_LAUNCH_CHECK();
    nmPass(2);
  } else {
    nmPass(0);
  }

  const bool a_k_fast = p.in_fs == 1;
  const bool b_n_fast = p.wn == 1;
  // the largest tile that still gives every SM a CTA
  auto ctas = [&](int t) {
    return (long long)((p.out_size + 16 * t - 1) / (16 * t)) * ((p.m + 16 * t - 1) / (16 * t));
  };
  const int T = ctas(4) >= n_sm ? 4 : (ctas(2) >= n_sm ? 2 : 1);
  const bool pcm = ioNeedsLineChain(p.io);
#define AB200_SIMT(TT, PCM)                                                                        \
  {                                                                                                \
    dim3 grid((p.out_size + 16 * TT - 1) / (16 * TT), (p.m + 16 * TT - 1) / (16 * TT));           \
    if (a_k_fast && b_n_fast) {                                                                    \
      AB200_CUDA(launchChained(mvmSimtKernel<true, true, TT, PCM>, grid, dim3(256), 0, stream, p));                             \
    } else if (a_k_fast) {                                                                         \
      AB200_CUDA(launchChained(mvmSimtKernel<true, false, TT, PCM>, grid, dim3(256), 0, stream, p));                            \
    } else if (b_n_fast) {                                                                         \
      AB200_CUDA(launchChained(mvmSimtKernel<false, true, TT, PCM>, grid, dim3(256), 0, stream, p));                            \
    } else {                                                                                       \
      AB200_CUDA(launchChained(mvmSimtKernel<false, false, TT, PCM>, grid, dim3(256), 0, stream, p));                           \
    }                                                                                              \
  }
  if (pcm && p.io.pos_neg != 0) {
    // separate passes: two sets of the line-chain accumulators, the 16-wide tile
    dim3 grid((p.out_size + 15) / 16, (p.m + 15) / 16);
    if (a_k_fast && b_n_fast) {
      AB200_CUDA(launchChained(mvmSimtKernel<true, true, 1, true, false, true>, grid, dim3(256), 0, stream, p));
    } else if (a_k_fast) {
      AB200_CUDA(launchChained(mvmSimtKernel<true, false, 1, true, false, true>, grid, dim3(256), 0, stream, p));
    } else if (b_n_fast) {
      AB200_CUDA(launchChained(mvmSimtKernel<false, true, 1, true, false, true>, grid, dim3(256), 0, stream, p));
    } else {
      AB200_CUDA(launchChained(mvmSimtKernel<false, false, 1, true, false, true>, grid, dim3(256), 0, stream, p));
    }
  } else if (pcm) { // the second accumulator doubles the registers of a thread: the 32-wide tile at most
    if (T >= 2) {
      AB200_SIMT(2, true)
    } else {
      AB200_SIMT(1, true)
    }
  } else if (T == 4) {
    AB200_SIMT(4, false)
  } else if (T == 2) {
    AB200_SIMT(2, false)
  } else {
    AB200_SIMT(1, false)
  }
#undef AB200_SIMT
  AB200_LAUNCH_CHECK();
}

void launchBmRerun(const MvmProblem &p, cudaStream_t stream) {
  if (p.backward || p.io.is_perfect || p.io.bm == AB200_BM_NONE) {
    return;
  }
  if (p.accumulate) {
    AB200_FATAL("bound management cannot be combined with accumulating outputs");
  }
  size_t smem = (size_t)p.in_size * sizeof(float);
  if (smem > 200 * 1024) {
    AB200_FATAL("bound management: x_size too large for the re-run kernel");
  }
  if (smem > 48 * 1024) {
    AB200_CUDA(cudaFuncSetAttribute(bmRerunKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    200 * 1024));
  }
  int blocks = p.m < 592 ? p.m : 592;
  AB200_CUDA(launchChained(bmRerunKernel, dim3(blocks), dim3(256), smem, stream, p));
  AB200_LAUNCH_CHECK();
}

void launchMvm(const MvmProblem &p, cudaStream_t stream) {
  if (p.m <= 0) {
    return;
  }
  launchMvmSimt(p, stream);
  launchBmRerun(p, stream);
}

// ---------------------------------------------------------------------------------------------
// Forward pass for callers that must not allocate.
//
// Some hosts hand the whole GPU to their own memory pool at start-up and forbid every later
// device allocation (an inference server's execute callback, a real-time control loop, a plugin
// whose contract says "no allocation after initialisation"); for them a cudaMalloc in the middle
// of a request either fails outright or stalls every stream of the device while the driver
// serialises it. The tile entry points grow their per-sample scratch with cudaMalloc on demand,
// so those callers get this variant: the same kernels, with the per-sample scratch (input scale,
// output factor, input norm, noise-management value, bound-management flag, two counters) living
// in a fixed array inside the library image. Every GPU that loads the library carries that array
// (about 320 KB) until the process exits.
//
// The array below is named from host code only as a *symbol*: its device address is looked up
// once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------------------------
constexpr int kNoAllocMaxBatch = AB200_NOALLOC_MAX_BATCH;
constexpr size_t kNoAllocBytes = (size_t)kNoAllocMaxBatch * 5 * sizeof(float) + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
static unsigned char *g_noalloc_ptr[kMaxDevices] = {nullptr};

static unsigned char *noAllocScratchForCurrentDevice() {
  int dev = -1;
  AB200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    AB200_FATAL("no-alloc forward: unsupported device index " << dev);
  }
  if (g_noalloc_ptr[dev] == nullptr) {
    // first call on this device: resolve the symbol to this device's address
    void *ptr = nullptr;
    AB200_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) {
      AB200_FATAL("no-alloc forward: scratch symbol has no device address");
    }
    g_noalloc_ptr[dev] = static_cast<unsigned char *>(ptr);
  }
  return g_noalloc_ptr[dev];
}

void forwardNoAlloc(const ab200_io_params &io_user, const float *w_dev_xd, int x_size, int d_size,
                    const float *x_dev, float *d_dev, int m_batch, uint64_t seed, uint32_t call,
                    cudaStream_t stream) {
  if (x_size <= 0 || d_size <= 0) {
    AB200_FATAL("no-alloc forward: tile sizes must be positive");
  }
  if (m_batch < 0) {
    AB200_FATAL("m_batch must be >= 0");
  }
  if (m_batch > kNoAllocMaxBatch) {
    AB200_FATAL("no-alloc forward: m_batch " << m_batch << " exceeds the built-in scratch ("
                                             << kNoAllocMaxBatch
                                             << " rows); split the batch or use ab200_tile_forward");
  }
  if (!w_dev_xd || (m_batch > 0 && (!x_dev || !d_dev))) {
    AB200_FATAL("no-alloc forward: null pointer");
  }
  if (m_batch == 0) {
    return;
  }
  if (!io_user.is_perfect && (io_user.out_noise_std > 0.0f || io_user.v_offset_std > 0.0f ||
                              io_user.r_series > 0.0f || io_user.out_nonlinearity > 0.0f)) {
    AB200_FATAL("no-alloc forward: per-line IO values (out_noise_std, v_offset_std, r_series, "
                "out_nonlinearity) need a tile, they belong to it");
  }
  unsigned char *base = noAllocScratchForCurrentDevice();
  MvmProblem p{};
  p.in = x_dev;
  p.in_ss = x_size;
  p.in_fs = 1;
  p.in_size = x_size;
  p.in_real = x_size;
  p.out = d_dev;
  p.out_ss = d_size;
  p.out_fs = 1;
  p.out_size = d_size;
  p.out_store = d_size;
  p.accumulate = 0;
  p.w = w_dev_xd;
  p.wk = d_size;
  p.wn = 1;
  p.m = m_batch;
  p.backward = 0;
  p.io = resolveIO(io_user, false);
  p.alpha = 1.0f;
  p.key.k0 = (uint32_t)seed;
  p.key.k1 = (uint32_t)(seed >> 32) ^ 0x5bd1e995u;
  p.call = call;
  p.noise_id = 0;
  float *f = reinterpret_cast<float *>(base);
  p.scale = f;
  p.factor = f + kNoAllocMaxBatch;
  p.vnorm = f + 2 * (size_t)kNoAllocMaxBatch;
  p.sval = f + 3 * (size_t)kNoAllocMaxBatch;
  p.flags = reinterpret_cast<int *>(f + 4 * (size_t)kNoAllocMaxBatch);
  p.bm_stats = reinterpret_cast<int *>(base + (size_t)kNoAllocMaxBatch * 5 * sizeof(float));
  // the array keeps what the previous call left: the first kernel zeroes the two counters and
  // rewrites the per-sample entries before anything reads them
  launchMvm(p, stream);
}

} // namespace ab200

namespace ab200 {
void setLastError(const char *msg);
}

extern "C" int ab200_mvm_forward_noalloc(const ab200_io_params *forward_io, const float *w_dev_xd,
                                         int x_size, int d_size, const float *x_dev, float *d_dev,
                                         int m_batch, uint64_t seed, uint32_t call, void *stream) {
  try {
    if (!forward_io) {
      AB200_FATAL("no-alloc forward: null IO parameters");
    }
    ab200::forwardNoAlloc(*forward_io, w_dev_xd, x_size, d_size, x_dev, d_dev, m_batch, seed, call,
                          (cudaStream_t)stream);
  } catch (const std::exception &e) {
    ab200::setLastError(e.what());
    return 1;
  }
  return 0;
}

namespace ab200 {
} // namespace ab200
