/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * C wrapper around the UNMODIFIED reference CPU tile (RPU::RPUPulsed<float>,
 * src/rpucuda/rpu_pulsed.h:23-125).  It is compiled together with the reference's own
 * sources, from where they lie, by oracle/Makefile into oracle/_ref/librpu_ref.so.  The
 * wrapper only translates the flat config structs of include/aihwkit_b200.h into the
 * reference's meta-parameter classes and forwards calls; all arithmetic is the reference's.
 *
 * Used by: tests/ (parity checks, golden-vector generation), bench.py's CPU-baseline legs.
 */
#include "aihwkit_b200.h"

#include "dense_bit_line_maker.h"
#include "rpu_buffered_transfer_device.h"
#include "rpu_chopped_transfer_device.h"
#include "rpu_dynamic_transfer_device.h"
#include "rpu_mixedprec_device.h"
#include "rpu_constantstep_device.h"
#include "rpu_expstep_device.h"
#include "rpu_linearstep_device.h"
#include "rpu_piecewisestep_device.h"
#include "rpu_powstep_device.h"
#include "rpu_pulsed.h"
#include "rpu_softbounds_reference_device.h"
#include "rpu_transfer_device.h"
#include "weight_modifier.h"

#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace RPU;

namespace {
thread_local std::string g_err;

void toIO(const ab200_io_params &s, IOMetaParameter<float> &io) {
  io.is_perfect = s.is_perfect != 0;
  io.noise_management = (NoiseManagementType)s.noise_management;
  io.bound_management = (BoundManagementType)s.bound_management;
  io.w_noise_type = (OutputWeightNoiseType)s.w_noise_type;
  io.bm_test_negative_bound = s.bm_test_negative_bound != 0;
  io.max_bm_factor = s.max_bm_factor;
  io.inp_sto_round = s.inp_sto_round != 0;
  io.out_sto_round = s.out_sto_round != 0;
  io.inp_bound = s.inp_bound;
  io.inp_res = s.inp_res;
  io.inp_noise = s.inp_noise;
  io.out_bound = s.out_bound;
  io.out_res = s.out_res;
  io.out_noise = s.out_noise;
  io.out_scale = s.out_scale;
  io.w_noise = s.w_noise;
  io.nm_thres = s.nm_thres;
  io.max_bm_res = s.max_bm_res;
  io.inp_asymmetry = s.inp_asymmetry;
  io.out_asymmetry = s.out_asymmetry;
  io.nm_assumed_wmax = s.nm_assumed_wmax;
  io.out_noise_std = s.out_noise_std;
  io.nm_decay = s.nm_decay;
  io.ir_drop = s.ir_drop;
  io.ir_drop_Gw_div_gmax = s.ir_drop_g_ratio;
  io.v_offset_std = s.v_offset_std;
  io.r_series = s.r_series;
  if (s.r_series_max_total > 0.0f) {
    io.r_series_max_total = s.r_series_max_total;
  }
  io.out_nonlinearity = s.out_nonlinearity;
  io.out_nonlinearity_std = s.out_nonlinearity_std;
  io.slope_calibration = s.slope_calibration;
  io.mv_type = s.mv_type == AB200_MV_POS_NEG_SEPARATE
                   ? AnalogMVType::PosNegSeparate
                   : (s.mv_type == AB200_MV_POS_NEG_SEPARATE_DIGITAL_SUM ? AnalogMVType::PosNegSeparateDigitalSum
                                                                         : AnalogMVType::OnePass);
}

void toUp(const ab200_update_params &s, PulsedUpdateMetaParameter<float> &up) {
  up.pulse_type = (PulseType)s.pulse_type;
  up.desired_BL = s.desired_bl;
  up.fixed_BL = s.fixed_bl != 0;
  up.update_management = s.update_management != 0;
  up.update_bl_management = s.update_bl_management != 0;
  up.sto_round = s.sto_round != 0;
  up.um_grad_scale = s.um_grad_scale;
  up.res = s.res;
  up.x_res_implicit = s.x_res_implicit;
  up.d_res_implicit = s.d_res_implicit;
}

void toDrift(const ab200_drift_params &s, DriftParameter<float> &d) {
  d.nu = s.nu;
  d.nu_dtod = s.nu_dtod;
  d.nu_std = s.nu_std;
  d.wg_ratio = s.wg_ratio != 0.0f ? s.wg_ratio : 1.0f;
  d.g_offset = s.g_offset;
  d.w_offset = s.w_offset;
  d.nu_k = s.nu_k;
  d.logG0 = s.log_g0;
  d.t0 = s.t0 > 0.0f ? s.t0 : 1.0f;
  d.reset_tol = s.reset_tol > 0.0f ? s.reset_tol : 1e-7f;
  d.w_read_std = s.w_read_std;
}

void toPulsedBase(const ab200_device_params &s, PulsedRPUDeviceMetaParameter<float> &p) {
  p.construction_seed = s.construction_seed;
  p.enforce_consistency = s.enforce_consistency != 0;
  p.dw_min_dtod_log_normal = s.dw_min_dtod_log_normal != 0;
  p.perfect_bias = s.perfect_bias != 0;
  p.dw_min = s.dw_min;
  p.dw_min_dtod = s.dw_min_dtod;
  p.dw_min_std = s.dw_min_std;
  p.w_min = s.w_min;
  p.w_min_dtod = s.w_min_dtod;
  p.w_max = s.w_max;
  p.w_max_dtod = s.w_max_dtod;
  p.up_down = s.up_down;
  p.up_down_dtod = s.up_down_dtod;
  p.lifetime = s.lifetime;
  p.lifetime_dtod = s.lifetime_dtod;
  p.diffusion = s.diffusion;
  p.diffusion_dtod = s.diffusion_dtod;
  p.reset = s.reset;
  p.reset_dtod = s.reset_dtod;
  p.reset_std = s.reset_std;
  toDrift(s.drift, p.drift);
}

std::unique_ptr<PulsedRPUDeviceMetaParameter<float>> makeSingle(const ab200_device_params &s) {
  switch (s.kind) {
  case AB200_DEVICE_CONSTANT_STEP: {
    auto p = std::make_unique<ConstantStepRPUDeviceMetaParameter<float>>();
    toPulsedBase(s, *p);
    return p;
  }
  case AB200_DEVICE_LINEAR_STEP:
  case AB200_DEVICE_SOFT_BOUNDS: {
    std::unique_ptr<LinearStepRPUDeviceMetaParameter<float>> p;
    if (s.kind == AB200_DEVICE_SOFT_BOUNDS) {
      p = std::make_unique<SoftBoundsRPUDeviceMetaParameter<float>>();
    } else {
      p = std::make_unique<LinearStepRPUDeviceMetaParameter<float>>();
      p->ls_decrease_up = s.ls_decrease_up;
      p->ls_decrease_down = s.ls_decrease_down;
      p->ls_decrease_up_dtod = s.ls_decrease_up_dtod;
      p->ls_decrease_down_dtod = s.ls_decrease_down_dtod;
      p->ls_allow_increasing_slope = s.ls_allow_increasing_slope != 0;
      p->ls_mean_bound_reference = s.ls_mean_bound_reference != 0;
    }
    p->ls_mult_noise = s.ls_mult_noise != 0;
    toPulsedBase(s, *p);
    return p;
  }
  case AB200_DEVICE_SOFT_BOUNDS_REFERENCE: {
    auto p = std::make_unique<SoftBoundsReferenceRPUDeviceMetaParameter<float>>();
    toPulsedBase(s, *p);
    p->mult_noise = s.mult_noise != 0;
    p->subtract_symmetry_point = s.subtract_symmetry_point != 0;
    p->slope_up_dtod = s.slope_up_dtod;
    p->slope_down_dtod = s.slope_down_dtod;
    p->reference_mean = s.reference_mean;
    p->reference_std = s.reference_std;
    return p;
  }
  case AB200_DEVICE_EXP_STEP: {
    auto p = std::make_unique<ExpStepRPUDeviceMetaParameter<float>>();
    toPulsedBase(s, *p);
    p->es_A_up = s.es_A_up;
    p->es_A_down = s.es_A_down;
    p->es_gamma_up = s.es_gamma_up;
    p->es_gamma_down = s.es_gamma_down;
    p->es_a = s.es_a;
    p->es_b = s.es_b;
    p->dw_min_std_add = s.dw_min_std_add;
    p->dw_min_std_slope = s.dw_min_std_slope;
    return p;
  }
  case AB200_DEVICE_POW_STEP: {
    auto p = std::make_unique<PowStepRPUDeviceMetaParameter<float>>();
    toPulsedBase(s, *p);
    p->ps_gamma = s.ps_gamma;
    p->ps_gamma_dtod = s.ps_gamma_dtod;
    p->ps_gamma_up_down = s.ps_gamma_up_down;
    p->ps_gamma_up_down_dtod = s.ps_gamma_up_down_dtod;
    return p;
  }
  case AB200_DEVICE_PIECEWISE_STEP: {
    auto p = std::make_unique<PiecewiseStepRPUDeviceMetaParameter<float>>();
    toPulsedBase(s, *p);
    p->piecewise_up_vec.assign(s.pw_up, s.pw_up + s.pw_n);
    p->piecewise_down_vec.assign(s.pw_down, s.pw_down + s.pw_n);
    return p;
  }
  default:
    throw std::runtime_error("ref_capi: unsupported device kind");
  }
}

struct RefTile {
  std::unique_ptr<RPUPulsed<float>> rpu;
  std::vector<std::string> names;
  PulsedUpdateMetaParameter<float> up;
  std::unique_ptr<DenseBitLineMaker<float>> dblm;
  std::unique_ptr<RNG<float>> rng;
  std::vector<int> indices; // the reference borrows the index array; the wrapper keeps it alive
};
} // namespace

#define REF_TRY try {
#define REF_CATCH                                                                                  \
  }                                                                                                \
  catch (const std::exception &e) {                                                                \
    g_err = e.what();                                                                              \
    return 1;                                                                                      \
  }                                                                                                \
  return 0;

extern "C" {

const char *ref_last_error(void) { return g_err.c_str(); }

int ref_tile_create(const ab200_tile_config *cfg, void **out) {
  REF_TRY
  PulsedMetaParameter<float> p;
  toIO(cfg->forward_io, p.f_io);
  toIO(cfg->backward_io, p.b_io);
  toUp(cfg->update, p.up);

  std::unique_ptr<AbstractRPUDeviceMetaParameter<float>> dp;
  if (cfg->device_kind == AB200_DEVICE_TRANSFER) {
    std::unique_ptr<TransferRPUDeviceMetaParameter<float>> tp;
    if (cfg->transfer.chopped) {
      std::unique_ptr<ChoppedTransferRPUDeviceMetaParameter<float>> cp;
      if (cfg->transfer.dynamic) {
        auto yp = std::make_unique<DynamicTransferRPUDeviceMetaParameter<float>>();
        yp->tail_weightening = cfg->transfer.tail_weightening;
        yp->buffer_cap = cfg->transfer.buffer_cap;
        yp->experimental_correct_accumulation = cfg->transfer.correct_accumulation != 0;
        cp = std::move(yp);
      } else {
        cp = std::make_unique<ChoppedTransferRPUDeviceMetaParameter<float>>();
      }
      cp->thres_scale = cfg->transfer.thres_scale;
      cp->step = cfg->transfer.step;
      cp->momentum = cfg->transfer.momentum;
      cp->forget_buffer = cfg->transfer.forget_buffer != 0;
      cp->in_chop_prob = cfg->transfer.in_chop_prob;
      cp->in_chop_random = cfg->transfer.in_chop_random != 0;
      cp->out_chop_prob = cfg->transfer.out_chop_prob;
      cp->correct_gradient_magnitudes = cfg->transfer.correct_gradient_magnitudes != 0;
      cp->auto_granularity = cfg->transfer.auto_granularity;
      cp->buffer_granularity = cfg->transfer.buffer_granularity;
      cp->no_buffer = cfg->transfer.no_buffer != 0;
      tp = std::move(cp);
    } else if (cfg->transfer.buffered) {
      auto bp = std::make_unique<BufferedTransferRPUDeviceMetaParameter<float>>();
      bp->thres_scale = cfg->transfer.thres_scale;
      bp->step = cfg->transfer.step;
      bp->momentum = cfg->transfer.momentum;
      bp->forget_buffer = cfg->transfer.forget_buffer != 0;
      tp = std::move(bp);
    } else {
      tp = std::make_unique<TransferRPUDeviceMetaParameter<float>>();
    }
    auto fast = makeSingle(cfg->device[0]);
    auto slow = makeSingle(cfg->device[1]);
    tp->appendVecPar(*fast);
    tp->appendVecPar(*slow);
    const ab200_transfer_params &t = cfg->transfer;
    tp->gamma = t.gamma;
    tp->transfer_every = t.transfer_every;
    tp->units_in_mbatch = t.units_in_mbatch != 0;
    tp->n_reads_per_transfer = t.n_reads_per_transfer;
    tp->fast_lr = t.fast_lr;
    tp->transfer_lr = t.transfer_lr;
    tp->scale_transfer_lr = t.scale_transfer_lr != 0;
    tp->scale_fast_lr = t.scale_fast_lr != 0;
    tp->transfer_columns = t.transfer_columns != 0;
    toIO(t.transfer_io, tp->transfer_io);
    toUp(t.transfer_up, tp->transfer_up);
    tp->construction_seed = cfg->device[0].construction_seed;
    dp = std::move(tp);
  } else if (cfg->device_kind == AB200_DEVICE_IDEAL) {
    auto sp = std::make_unique<SimpleRPUDeviceMetaParameter<float>>();
    sp->construction_seed = cfg->device[0].construction_seed;
    sp->lifetime = cfg->device[0].lifetime;
    sp->diffusion = cfg->device[0].diffusion;
    sp->reset_std = cfg->device[0].reset_std;
    toDrift(cfg->device[0].drift, sp->drift);
    dp = std::move(sp);
  } else {
    ab200_device_params d = cfg->device[0];
    d.kind = cfg->device_kind;
    dp = makeSingle(d);
    if (cfg->mixed.enabled) {
      const ab200_mixedprec_params &m = cfg->mixed;
      auto mp = std::make_unique<MixedPrecRPUDeviceMetaParameter<float>>();
      mp->setDevicePar(*dp);
      mp->transfer_every = m.transfer_every;
      mp->n_rows_per_transfer = m.n_rows_per_transfer;
      mp->random_row = m.random_row != 0;
      mp->granularity = m.granularity;
      mp->n_x_bins = m.n_x_bins;
      mp->n_d_bins = m.n_d_bins;
      mp->stoc_round_x = m.stoc_round_x != 0;
      mp->stoc_round_d = m.stoc_round_d != 0;
      mp->transfer_lr = m.transfer_lr;
      mp->construction_seed = cfg->device[0].construction_seed;
      dp = std::move(mp);
    }
  }

  auto t = new RefTile();
  t->rpu.reset(p.createRPUArray(cfg->x_size, cfg->d_size, dp.get()));
  std::vector<float> zeros((size_t)cfg->x_size * cfg->d_size, 0.0f);
  t->rpu->setWeights(zeros.data());
  t->rpu->getDeviceParameterNames(t->names);
  t->up = p.up;
  t->up.initialize();
  if (cfg->seed) {
    t->rpu->setRandomSeed((unsigned int)cfg->seed);
  }
  *out = t;
  REF_CATCH
}

int ref_tile_destroy(void *h) {
  delete static_cast<RefTile *>(h);
  return 0;
}

int ref_tile_set_seed(void *h, uint64_t seed) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->setRandomSeed((unsigned int)seed);
  REF_CATCH
}

int ref_tile_set_learning_rate(void *h, float lr) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->setLearningRate(lr);
  REF_CATCH
}

int ref_tile_set_weights(void *h, const float *w) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->setWeights(w);
  REF_CATCH
}

int ref_tile_get_weights(void *h, float *w) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->getWeights(w);
  REF_CATCH
}

int ref_tile_hidden_parameter_count(void *h) {
  return (int)static_cast<RefTile *>(h)->names.size();
}

const char *ref_tile_hidden_parameter_name(void *h, int i) {
  auto *t = static_cast<RefTile *>(h);
  if (i < 0 || i >= (int)t->names.size()) {
    return "";
  }
  return t->names[i].c_str();
}

int ref_tile_get_hidden_parameters(void *h, float *out) {
  REF_TRY
  auto *t = static_cast<RefTile *>(h);
  size_t sz = (size_t)t->rpu->getXSize() * t->rpu->getDSize();
  std::vector<float *> ptrs(t->names.size());
  for (size_t i = 0; i < ptrs.size(); i++) {
    ptrs[i] = out + i * sz;
  }
  t->rpu->getDeviceParameter(ptrs);
  REF_CATCH
}

int ref_tile_set_hidden_parameters(void *h, const float *in) {
  REF_TRY
  auto *t = static_cast<RefTile *>(h);
  size_t sz = (size_t)t->rpu->getXSize() * t->rpu->getDSize();
  std::vector<float *> ptrs(t->names.size());
  for (size_t i = 0; i < ptrs.size(); i++) {
    ptrs[i] = const_cast<float *>(in) + i * sz;
  }
  t->rpu->setDeviceParameter(ptrs);
  REF_CATCH
}

int ref_tile_forward(
    void *h, const float *x, float *d, int bias, int m, int x_trans, int d_trans, int is_test) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->forward(x, d, bias != 0, m, x_trans != 0, d_trans != 0,
                                           is_test != 0);
  REF_CATCH
}

int ref_tile_backward(void *h, const float *d, float *x, int bias, int m, int d_trans, int x_trans) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->backward(d, x, bias != 0, m, d_trans != 0, x_trans != 0);
  REF_CATCH
}

int ref_tile_update(
    void *h, const float *x, const float *d, int bias, int m, int x_trans, int d_trans) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->update(x, d, bias != 0, m, x_trans != 0, d_trans != 0);
  REF_CATCH
}

/* DenseBitLineMaker<float>::makeCoincidences (src/rpucuda/dense_bit_line_maker.cpp:266-331):
   signed counts [d][x] of one sample for MeanCount / DeterministicImplicit. */
int ref_tile_coincidences(void *h, const float *x, const float *d, float lr, float dw_min,
                          int32_t *counts) {
  REF_TRY
  auto *t = static_cast<RefTile *>(h);
  int xs = t->rpu->getXSize(), ds = t->rpu->getDSize();
  if (!t->dblm) {
    t->dblm = std::make_unique<DenseBitLineMaker<float>>(xs, ds);
    t->rng = std::make_unique<RNG<float>>(1);
  }
  int xnoz = 0, dnoz = 0;
  int *c = t->dblm->makeCoincidences(x, 1, xnoz, d, 1, dnoz, t->rng.get(), lr, dw_min, t->up);
  std::memcpy(counts, c, sizeof(int) * (size_t)xs * ds);
  REF_CATCH
}

/* Indexed (im2col-free) convolution interface, RPUSimple<T>::setMatrixIndices / forwardIndexed /
   backwardIndexed / updateIndexed (src/rpucuda/rpu.h:452-478, src/rpucuda/rpu.cpp:1117-1239). */
int ref_tile_set_matrix_indices(void *h, const int *indices, long long n) {
  REF_TRY
  auto *t = static_cast<RefTile *>(h);
  t->indices.assign(indices, indices + n);
  t->rpu->setMatrixIndices(t->indices.data());
  REF_CATCH
}

int ref_tile_forward_indexed(void *h, const float *x, float *d, long long total_input_size,
                             int m_batch, int dim3, int trans, int is_test) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->forwardIndexed(x, d, (int)total_input_size, m_batch, dim3,
                                                 trans != 0, is_test != 0);
  REF_CATCH
}

int ref_tile_backward_indexed(void *h, const float *d, float *x, long long total_output_size,
                              int m_batch, int dim3, int trans) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->backwardIndexed(d, x, (int)total_output_size, m_batch, dim3,
                                                  trans != 0);
  REF_CATCH
}

int ref_tile_update_indexed(void *h, const float *x, const float *d, long long total_input_size,
                            int m_batch, int dim3, int trans) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->updateIndexed(x, d, (int)total_input_size, m_batch, dim3,
                                                trans != 0);
  REF_CATCH
}

/* Weight operations between updates (src/rpucuda/rpu_pulsed.cpp:189-284). */
int ref_tile_decay_weights(void *h, float alpha, int bias_no_decay) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->decayWeights(alpha, bias_no_decay != 0);
  REF_CATCH
}

/* The per-line IO vectors the reference drew at construction, out of its extra state
 * (ForwardBackwardPass::dumpExtra, src/rpucuda/rpu_forward_backward_pass.cpp:63-82). Returns the
 * number of values (0: the vector is not in use); at most `n` are copied. */
int ref_tile_get_io_vector(void *h, int backward, int which, float *values, int n) {
  try {
    RPU::state_t st;
    static_cast<RefTile *>(h)->rpu->dumpExtra(st, "rpu");
    const char *names[3] = {"v_offset", "out_nonlinearity", "out_noise_values"};
    if (which < 0 || which > 2) {
      return -1;
    }
    const std::string suffix = std::string("fb_pass.") + (backward ? "bwd." : "fwd.") + names[which];
    for (const auto &kv : st) {
      const std::string &k = kv.first;
      if (k.size() >= suffix.size() && k.compare(k.size() - suffix.size(), suffix.size(), suffix) == 0) {
        const int cnt = (int)kv.second.size();
        for (int i = 0; i < cnt && i < n; i++) {
          values[i] = (float)kv.second[(size_t)i];
        }
        return cnt;
      }
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

int ref_tile_modify_weights(void *h, const ab200_weight_modifier_params *s) {
  REF_TRY
  WeightModifierParameter<float> wm;
  wm.type = (WeightModifierType)s->type;
  wm.sto_round = s->sto_round != 0;
  wm.enable_during_test = s->enable_during_test != 0;
  wm.copy_last_column = s->copy_last_column != 0;
  wm.rel_to_actual_wmax = s->rel_to_actual_wmax != 0;
  wm.std_dev = s->std_dev;
  wm.res = s->res;
  wm.dorefa_clip = s->dorefa_clip;
  wm.pdrop = s->pdrop;
  wm.assumed_wmax = s->assumed_wmax;
  wm.g_max = s->g_max;
  wm.coeffs.assign(s->coeffs, s->coeffs + s->n_coeffs);
  static_cast<RefTile *>(h)->rpu->modifyFBWeights(wm);
  REF_CATCH
}

int ref_tile_drift_weights(void *h, float time_since_last_call) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->driftWeights(time_since_last_call);
  REF_CATCH
}

int ref_tile_diffuse_weights(void *h) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->diffuseWeights();
  REF_CATCH
}

int ref_tile_clip_weights(void *h, int clip_type, float fixed_value, float sigma) {
  REF_TRY
  WeightClipParameter wc;
  wc.type = (WeightClipType)clip_type;
  wc.fixed_value = fixed_value;
  wc.sigma = sigma;
  static_cast<RefTile *>(h)->rpu->clipWeights(wc);
  REF_CATCH
}

int ref_tile_reset_columns(void *h, int start_col, int n_cols, float reset_prob) {
  REF_TRY
  static_cast<RefTile *>(h)->rpu->resetCols(start_col, n_cols, reset_prob);
  REF_CATCH
}

} // extern "C"
