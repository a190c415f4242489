// Host side of the analog tile: configuration, per-element device parameters, weight access and
// the sequencing of forward / backward / update (including Tiki-Taka transfers).
#include "tile.h"
#include "tc_engine.h"

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <random>

namespace ab200 {

static std::atomic<uint64_t> g_launches{0};
void countLaunch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launchCount() { return g_launches.load(std::memory_order_relaxed); }

static std::atomic<int> g_mvm_path{0};
void setMvmPath(int mode) { g_mvm_path.store(mode); }
int mvmPath() { return g_mvm_path.load(); }

// detail::checkRes (src/rpucuda/rpu_pulsed_meta_parameter.cpp:26-29)
static float checkRes(float res) {
  float r = res < 0.0f ? 0.0f : res;
  return r > 1.0f ? 1.0f / r : r;
}

bool pdlEnabled() {
  static const bool on = [] {
    const char *e = getenv("AB200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

IOEff resolveIO(const ab200_io_params &io, bool backward, bool plain_only) {
  // IOMetaParameter::initializeForForward / Backward (rpu_pulsed_meta_parameter.cpp:40-128)
  IOEff e;
  e.is_perfect = io.is_perfect;
  e.nm = io.noise_management;
  e.bm = backward ? AB200_BM_NONE : io.bound_management;
  e.w_noise_type = io.w_noise_type;
  e.bm_test_negative_bound = io.bm_test_negative_bound;
  e.max_bm_factor = io.max_bm_factor;
  e.max_bm_res = io.max_bm_res;
  e.res_out = checkRes(io.out_res) * (2.0f * io.out_bound);
  e.res_in = checkRes(io.inp_res) * (2.0f * io.inp_bound);
  e.nm_thres = io.noise_management == AB200_NM_NONE ? 0.0f : io.nm_thres;
  e.out_bound = io.out_bound <= 0.0f ? std::numeric_limits<float>::infinity() : io.out_bound;
  e.inp_bound = io.inp_bound <= 0.0f ? std::numeric_limits<float>::infinity() : io.inp_bound;
  e.out_noise = io.out_noise;
  e.out_noise_std = io.out_noise_std > 0.0f ? io.out_noise_std : 0.0f;
  e.out_scale = io.out_scale;
  e.w_noise = io.w_noise;
  e.nm_assumed_wmax = io.nm_assumed_wmax;
  e.nm_decay = io.nm_decay;
  e.ir_drop = io.ir_drop > 0.0f ? io.ir_drop : 0.0f;
  e.ir_g_ratio = io.ir_drop_g_ratio;
  e.v_offset_std = io.v_offset_std > 0.0f ? io.v_offset_std : 0.0f;
  e.r_series = io.r_series > 0.0f ? io.r_series : 0.0f;
  e.r_series_max = io.r_series_max_total > 0.0f ? io.r_series_max_total : std::numeric_limits<float>::max();
  e.out_nl = io.out_nonlinearity;
  e.out_nl_std = io.out_nonlinearity_std;
  e.slope_calibration = io.slope_calibration;
  e.inp_noise = io.inp_noise;
  e.inp_asym = 1.0f - io.inp_asymmetry;
  e.out_asym = 1.0f - io.out_asymmetry;
  e.inp_sto_round = io.inp_sto_round;
  e.out_sto_round = io.out_sto_round;
  e.pos_neg = 0;
  if (!io.is_perfect && io.mv_type != AB200_MV_ONE_PASS) {
    if (io.mv_type != AB200_MV_POS_NEG_SEPARATE && io.mv_type != AB200_MV_POS_NEG_SEPARATE_DIGITAL_SUM) {
      AB200_FATAL("AnalogMVType not implemented.");
    }
    if (plain_only) {
      AB200_FATAL("separate passes for negative and positive inputs are not implemented for the "
                  "read-out of a transfer");
    }
    e.pos_neg = io.mv_type == AB200_MV_POS_NEG_SEPARATE ? 1 : 2;
  }
  if (!io.is_perfect) {
    if (io.noise_management != AB200_NM_NONE && io.inp_bound != 1.0f) {
      AB200_FATAL((backward ? "Backward noise managment expects input bound==1"
                            : "Forward noise managment expects bound==1"));
    }
    if (io.noise_management < AB200_NM_NONE || io.noise_management > AB200_NM_AVERAGE_ABS_MAX_SINGLE_VALUE) {
      AB200_FATAL("Noise Management type not implemented!");
    }
    if (plain_only && (io.noise_management == AB200_NM_AVERAGE_ABS_MAX ||
                       io.noise_management == AB200_NM_AVERAGE_ABS_MAX_SINGLE_VALUE)) {
      AB200_FATAL("running-average noise management is not implemented for the read-out of a transfer");
    }
    if (e.ir_drop > 0.0f && !(io.ir_drop_g_ratio > 0.0f)) {
      AB200_FATAL("ir_drop needs a positive ir_drop_g_ratio");
    }
    if (plain_only && (e.ir_drop > 0.0f || e.v_offset_std > 0.0f || e.r_series > 0.0f ||
                       io.out_nonlinearity > 0.0f)) {
      AB200_FATAL("IR drop / voltage offsets / output non-linearity are not implemented for the "
                  "read-out of a transfer");
    }
    if (plain_only && ((io.w_noise_type == AB200_WNOISE_PCM_READ && io.w_noise > 0.0f) ||
                       io.out_noise_std > 0.0f)) {
      AB200_FATAL("PCMRead weight noise / out_noise_std are not implemented for the read-out of "
                  "a transfer");
    }
    if (plain_only && (io.inp_noise != 0.0f || io.inp_sto_round || io.out_sto_round ||
                       io.inp_asymmetry != 0.0f || io.out_asymmetry != 0.0f)) {
      AB200_FATAL("inp_noise / stochastic rounding / asymmetry are not implemented for the "
                  "read-out of a transfer");
    }
  }
  return e;
}

UpEff resolveUp(const ab200_update_params &up) {
  UpEff e;
  e.pulse_type = up.pulse_type;
  e.desired_bl = up.desired_bl;
  e.fixed_bl = up.fixed_bl;
  e.update_bl_management = up.update_bl_management;
  // "always turn on UM for UBL management" (rpu_pulsed_meta_parameter.cpp:139-141)
  e.update_management = up.update_management || up.update_bl_management;
  e.um_grad_scale = up.um_grad_scale;
  e.res = checkRes(up.res);
  e.x_res_implicit = checkRes(up.x_res_implicit);
  e.d_res_implicit = checkRes(up.d_res_implicit);
  if (up.pulse_type == AB200_PULSE_STOCHASTIC) {
    // Separate trains for positive and negative x-lines (generateCountsPN,
    // sparse_bit_line_maker.cpp:147-197, applied one sign group after the other,
    // rpu_weight_updater.cpp:262-286): a line has one sign per sample, so it carries exactly one
    // Bernoulli train either way, and a weight receives a pulse in slot k iff both its lines
    // pulse in k - the same law per weight, in the same per-weight order, as the compressed type.
    e.pulse_type = AB200_PULSE_STOCHASTIC_COMPRESSED;
  }
  e.sto_round = up.sto_round != 0;
  return e;
}

// ---------------------------------------------------------------------------------------------
// Per-element device parameters, drawn on the host in the reference's order of draws
// (RealWorldRNG = std::default_random_engine + std::normal_distribution<float>,
//  src/rpucuda/rng.h:45-61; PulsedRPUDevice::populate, rpu_pulsed_device.cpp:594-733;
//  LinearStepRPUDevice::populate, rpu_linearstep_device.cpp:21-74;
//  SoftBoundsReferenceRPUDevice::populate, rpu_softbounds_reference_device.cpp:21-68).
// ---------------------------------------------------------------------------------------------
namespace {
struct HostRNG {
  explicit HostRNG(unsigned int seed) {
    if (!seed) {
      seed = (unsigned int)std::chrono::high_resolution_clock::now().time_since_epoch().count();
    }
    gen = std::default_random_engine(seed);
  }
  float gauss() { return nd(gen); }
  float uniform() { return ud(gen); }
  std::default_random_engine gen;
  std::uniform_real_distribution<float> ud{0.0f, 1.0f};
  std::normal_distribution<float> nd{0.0f, 1.0f};
};

std::vector<std::string> deviceNames(int kind) {
  std::vector<std::string> n = {"max_bound",    "min_bound",       "dwmin_up",   "dwmin_down",
                                "decay_scales", "diffusion_rates", "reset_bias", "drift_nu"};
  if (kind == AB200_DEVICE_LINEAR_STEP || kind == AB200_DEVICE_SOFT_BOUNDS) {
    n.push_back("slope_up");
    n.push_back("slope_down");
  } else if (kind == AB200_DEVICE_SOFT_BOUNDS_REFERENCE) {
    n.push_back("reference");
  } else if (kind == AB200_DEVICE_POW_STEP) {
    n.push_back("gamma_up");
    n.push_back("gamma_down");
  }
  return n;
}

// calcWeightGranularity of the device kinds: the weight change the pulse-count learning rate is
// measured in (rpu_pulsed_device.h: dw_min; rpu_expstep_device.h:43-55; rpu_powstep_device.h:33;
// rpu_piecewisestep_device.h:34-39)
float weightGranularity(const ab200_device_params &par, int kind) {
  if (kind == AB200_DEVICE_EXP_STEP) {
    // the step at w = 0 (the reference averages the down step with itself)
    const float down_bias = par.up_down > 0.0f ? -par.up_down : 0.0f;
    const float scale_down = (down_bias + 1.0f) * par.dw_min;
    const float z = par.es_b;
    const float dw_down = scale_down * fmaxf(1.0f - par.es_A_down * expf(par.es_gamma_down * (-z)), 0.0f);
    const float g = fmaxf((dw_down + dw_down) / 2.0f, 0.0f);
    return g > 0.0f ? g : par.dw_min;
  }
  if (kind == AB200_DEVICE_PIECEWISE_STEP && par.pw_n > 0 && par.pw_n <= AB200_PIECEWISE_MAX_NODES) {
    return par.dw_min * par.pw_up[par.pw_n / 2];
  }
  if (kind == AB200_DEVICE_POW_STEP) {
    return par.dw_min * powf(0.5f, par.ps_gamma);
  }
  return par.dw_min;
}

void populateDevice(const ab200_device_params &par, int kind, int x_size, int d_size, HostRNG &rng,
                    DeviceStore &ds) {
  ds.kind = kind;
  ds.dw_min = weightGranularity(par, kind);
  ds.dw_min_std = par.dw_min_std;
  if (kind == AB200_DEVICE_EXP_STEP) {
    ds.es0 = make_float4(par.es_a, par.es_b, par.es_A_up, par.es_A_down);
    ds.es1 = make_float4(par.es_gamma_up, par.es_gamma_down, par.dw_min_std_add, par.dw_min_std_slope);
  }
  if (kind == AB200_DEVICE_PIECEWISE_STEP) {
    // PiecewiseStepRPUDeviceMetaParameter::initialize / calcWeightGranularity
    // (rpu_piecewisestep_device.h:34-50)
    if (par.pw_n <= 0) {
      AB200_FATAL("piecewise_up_vec and piecewise_down_vec needs to have some contents.");
    }
    if (par.pw_n > AB200_PIECEWISE_MAX_NODES) {
      AB200_FATAL("PiecewiseStep: at most " << AB200_PIECEWISE_MAX_NODES << " nodes per direction");
    }
    ds.pw_n = par.pw_n;
    ds.pw_host.assign(par.pw_up, par.pw_up + par.pw_n);
    ds.pw_host.insert(ds.pw_host.end(), par.pw_down, par.pw_down + par.pw_n);
  }
  ds.mult_noise = kind == AB200_DEVICE_SOFT_BOUNDS_REFERENCE ? par.mult_noise : par.ls_mult_noise;
  ds.names = deviceNames(kind);
  const size_t size = (size_t)x_size * d_size;
  ds.host.assign(ds.names.size() * size, 0.0f);
  float *wmax = &ds.host[0 * size], *wmin = &ds.host[1 * size], *sup = &ds.host[2 * size],
        *sdown = &ds.host[3 * size], *decay = &ds.host[4 * size], *diffusion = &ds.host[5 * size],
        *reset_bias0 = &ds.host[6 * size];
  ds.reset_std = par.reset_std;

  if (par.w_min > 0.0f || par.w_max < 0.0f) {
    AB200_FATAL("The closed interval [w_min,w_max] needs to contain 0.");
  }
  const float up_bias = par.up_down > 0.0f ? 0.0f : par.up_down;
  const float down_bias = par.up_down > 0.0f ? -par.up_down : 0.0f;

  if (par.drift.nu > 0.0f) {
    // the exponents of the drift are the first draws (SimpleRPUDevice::populate ->
    // WeightDrifter::populate, rpu_simple_device.cpp:172-181, weight_drifter.cpp:57-65)
    float *nu = &ds.host[7 * size];
    for (size_t k = 0; k < size; k++) {
      nu[k] = par.drift.nu + par.drift.nu_dtod * par.drift.nu * rng.gauss();
    }
  }

  for (int j = 0; j < x_size; ++j) {
    for (int i = 0; i < d_size; ++i) {
      const size_t k = (size_t)i * x_size + j;
      wmax[k] = par.w_max * (1.0f + par.w_max_dtod * rng.gauss());
      wmin[k] = par.w_min * (1.0f + par.w_min_dtod * rng.gauss());
      float gain = par.dw_min_dtod_log_normal ? expf(par.dw_min_dtod * rng.gauss())
                                              : (1.0f + par.dw_min_dtod * rng.gauss());
      float r = par.up_down_dtod * rng.gauss();
      sup[k] = (up_bias + gain + r) * par.dw_min;
      sdown[k] = (down_bias + gain - r) * par.dw_min;
      if (par.enforce_consistency) {
        sup[k] = fabsf(sup[k]);
        sdown[k] = fabsf(sdown[k]);
        if (wmin[k] > wmax[k]) {
          std::swap(wmin[k], wmax[k]);
        }
        wmax[k] = fabsf(wmax[k]);
        wmin[k] = -fabsf(wmin[k]);
      } else if (wmin[k] > wmax[k]) {
        float m = wmax[k] + (wmin[k] - wmax[k]) / 2.0f;
        wmax[k] = m;
        wmin[k] = m;
      }
      // corrupt-device draw (probability 0 here, but the draw is part of the sequence)
      (void)rng.uniform();
      if (par.perfect_bias && j == x_size - 1) {
        sup[k] = par.dw_min;
        sdown[k] = par.dw_min;
        wmin[k] = 100.0f * par.w_min;
        wmax[k] = 100.0f * par.w_max;
      }
      // diffusion rate, reset bias, decay scale (rpu_pulsed_device.cpp:704-731): the first two
      // always draw, the decay scale only with a lifetime
      diffusion[k] = fabsf(par.diffusion * (1.0f + par.diffusion_dtod * rng.gauss()));
      reset_bias0[k] = par.reset + par.reset_dtod * rng.gauss();
      if (par.lifetime > 0.0f) {
        float t = par.lifetime * (1.0f + par.lifetime_dtod * rng.gauss());
        decay[k] = t > 1.0f ? 1.0f - 1.0f / t : 0.0f;
      } else {
        decay[k] = 1.0f;
      }
    }
  }

  if (kind == AB200_DEVICE_LINEAR_STEP || kind == AB200_DEVICE_SOFT_BOUNDS) {
    float *slope_up = &ds.host[8 * size], *slope_down = &ds.host[9 * size];
    for (int i = 0; i < d_size; ++i) {
      for (int j = 0; j < x_size; ++j) {
        const size_t k = (size_t)i * x_size + j;
        float du = par.ls_decrease_up + par.ls_decrease_up_dtod * rng.gauss();
        float dd = par.ls_decrease_down + par.ls_decrease_down_dtod * rng.gauss();
        if (!par.ls_allow_increasing_slope) {
          du = fabsf(du);
          dd = fabsf(dd);
        }
        float ref_up = par.ls_mean_bound_reference ? par.w_max : wmax[k];
        float ref_down = par.ls_mean_bound_reference ? par.w_min : wmin[k];
        slope_up[k] = ref_up != 0.0f ? -du * sup[k] / ref_up : 0.0f;
        slope_down[k] = ref_down != 0.0f ? -dd * sdown[k] / ref_down : 0.0f;
      }
    }
  } else if (kind == AB200_DEVICE_POW_STEP) {
    // PowStepRPUDevice::populate (rpu_powstep_device.cpp:21-51)
    float *gamma_up = &ds.host[8 * size], *gamma_down = &ds.host[9 * size];
    const float g_up_bias = par.ps_gamma_up_down > 0.0f ? 0.0f : par.ps_gamma_up_down;
    const float g_down_bias = par.ps_gamma_up_down > 0.0f ? -par.ps_gamma_up_down : 0.0f;
    for (int i = 0; i < d_size; ++i) {
      for (int j = 0; j < x_size; ++j) {
        const size_t k = (size_t)i * x_size + j;
        const float gain = 1.0f + par.ps_gamma_dtod * rng.gauss();
        const float r = par.ps_gamma_up_down_dtod * rng.gauss();
        gamma_up[k] = (g_up_bias + gain + r) * par.ps_gamma;
        gamma_down[k] = (g_down_bias + gain - r) * par.ps_gamma;
        if (par.enforce_consistency) {
          gamma_up[k] = fabsf(gamma_up[k]);
          gamma_down[k] = fabsf(gamma_down[k]);
        }
      }
    }
  } else if (kind == AB200_DEVICE_SOFT_BOUNDS_REFERENCE) {
    float *reference = &ds.host[8 * size], *reset_bias = &ds.host[6 * size];
    for (int i = 0; i < d_size; ++i) {
      for (int j = 0; j < x_size; ++j) {
        const size_t k = (size_t)i * x_size + j;
        float w_min = wmin[k], w_max = wmax[k];
        if (w_max > 0.0f && w_min < 0.0f) {
          float slope_down = -sdown[k] / w_min;
          slope_down *= fabsf(1.0f + par.slope_down_dtod * rng.gauss());
          float slope_up = sup[k] / w_max;
          slope_up *= fabsf(1.0f + par.slope_up_dtod * rng.gauss());
          w_max = sup[k] / slope_up;
          w_min = -sdown[k] / slope_down;
          wmax[k] = w_max;
          wmin[k] = w_min;
        }
        reference[k] = par.reference_mean + par.reference_std * rng.gauss();
        if (par.subtract_symmetry_point && w_max > 0.0f && w_min < 0.0f) {
          float sp = (sup[k] - sdown[k]) / (sup[k] / w_max - sdown[k] / w_min);
          reference[k] += sp;
          reset_bias[k] += sp;
        }
      }
    }
  }
}
} // namespace

void Tile::populateHost() {
  if (cfg_.device_kind == AB200_DEVICE_IDEAL) {
    n_dev_ = 1;
    dev_[0].kind = AB200_DEVICE_IDEAL;
    return;
  }
  HostRNG rng(cfg_.device[0].construction_seed);
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    n_dev_ = 2;
    for (int k = 0; k < 2; k++) {
      int kind = cfg_.device[k].kind;
      if ((kind < AB200_DEVICE_CONSTANT_STEP || kind > AB200_DEVICE_SOFT_BOUNDS_REFERENCE) &&
          kind != AB200_DEVICE_EXP_STEP && kind != AB200_DEVICE_POW_STEP &&
          kind != AB200_DEVICE_PIECEWISE_STEP) {
        AB200_FATAL("Transfer: unit cell device kind not implemented");
      }
      populateDevice(cfg_.device[k], kind, x_size_, d_size_, rng, dev_[k]);
    }
  } else {
    n_dev_ = 1;
    populateDevice(cfg_.device[0], cfg_.device_kind, x_size_, d_size_, rng, dev_[0]);
  }
}

Tile::Tile(const ab200_tile_config &cfg, int cuda_device) : cfg_(cfg) {
  x_size_ = cfg.x_size;
  d_size_ = cfg.d_size;
  if (x_size_ <= 0 || d_size_ <= 0) {
    AB200_FATAL("tile sizes must be positive");
  }
  f_io_ = resolveIO(cfg.forward_io, false);
  b_io_ = resolveIO(cfg.backward_io, true);
  up_ = resolveUp(cfg.update);
  if (cfg.device_kind < AB200_DEVICE_IDEAL || cfg.device_kind > AB200_DEVICE_PIECEWISE_STEP) {
    AB200_FATAL("device kind not implemented");
  }
  if (cfg.device[0].count_pulses || cfg.device[1].count_pulses) {
    if (cfg.device_kind == AB200_DEVICE_IDEAL || cfg.device_kind == AB200_DEVICE_TRANSFER || cfg.mixed.enabled) {
      AB200_FATAL("count_pulses is implemented for single pulsed devices only");
    }
  }
  if (cfg.mixed.enabled) {
    const ab200_mixedprec_params &mp = cfg.mixed;
    if (cfg.device_kind == AB200_DEVICE_IDEAL || cfg.device_kind == AB200_DEVICE_TRANSFER) {
      AB200_FATAL("MixedPrec: expects a pulsed analog device in device[0]");
    }
    if ((mp.n_x_bins > 0) != (mp.n_d_bins > 0)) {
      AB200_FATAL("MixedPrec: quantising only one of x and d is not implemented (set both n_x_bins and "
                  "n_d_bins, or neither)");
    }
    if (mp.transfer_every < 0) {
      AB200_FATAL("MixedPrec: transfer_every must not be negative");
    }
  }
  if (cfg.device_kind == AB200_DEVICE_TRANSFER) {
    const ab200_transfer_params &t = cfg.transfer;
    if (t.gamma != 0.0f) {
      AB200_FATAL("Transfer: only gamma = 0 (fully hidden fast tile) is implemented");
    }
    if (!t.transfer_columns) {
      AB200_FATAL("Transfer: row transfer is not implemented");
    }
    if (t.n_reads_per_transfer < 0) {
      AB200_FATAL("Transfer: n_reads_per_transfer must be >= 0");
    }
    if (t.chopped) {
      // ChoppedTransferRPUDeviceMetaParameter::checkSupported (rpu_chopped_transfer_device.cpp:66-88)
      if (!t.buffered) {
        AB200_FATAL("ChoppedTransfer: expects the buffered transfer parameters (buffered = 1)");
      }
      if (t.n_reads_per_transfer != 1) {
        AB200_FATAL("In / out chopper not implemented the given parameters. \nRequired: n_devices==2, "
                    "n_reads_per_transfer==1, random_selection=false).\n");
      }
      if (t.transfer_every < 0.0f) {
        AB200_FATAL("ChoppedTransfer: the automatic transfer period is not implemented");
      }
    }
    if (t.dynamic) {
      // DynamicTransferRPUDeviceMetaParameter::checkSupported (rpu_dynamic_transfer_device.cpp:38-49)
      if (!t.chopped) {
        AB200_FATAL("DynamicTransfer: expects the chopped transfer parameters (chopped = 1)");
      }
      if (t.in_chop_prob <= 0.0f) {
        AB200_FATAL("In chopper prob needs to be positive.");
      }
    }
    // transfer IO: noise and bound management are turned off (rpu_transfer_device.cpp:208-217)
    ab200_io_params tio = t.transfer_io;
    tio.noise_management = AB200_NM_NONE;
    tio.bound_management = AB200_BM_NONE;
    t_io_ = resolveIO(tio, false, /*plain_only=*/true);
    t_up_ = resolveUp(t.transfer_up);
  }
  setSeed(cfg.seed);
  populateHost();
  host_w_dx_.assign((size_t)x_size_ * d_size_, 0.0f);
  if (cuda_device >= 0) {
    toDevice(cuda_device);
  }
}

void Tile::setSeed(uint64_t seed) {
  if (seed == 0) {
    seed = (uint64_t)std::chrono::high_resolution_clock::now().time_since_epoch().count();
  }
  key_.k0 = (uint32_t)seed;
  key_.k1 = (uint32_t)(seed >> 32) ^ 0x5bd1e995u;
  fwd_calls_ = bwd_calls_ = upd_calls_ = transfer_calls_ = 0;
}

// ---------------------------------------------------------------------------------------------
// extra state
// ---------------------------------------------------------------------------------------------
namespace {
const char *const kExtraNames[] = {
    "learning_rate",                           // RPUSimple (rpu.cpp:438)
    "rpu_device.current_update_idx",           // VectorRPUDevice
    "rpu_device.current_slice_indices",        // TransferRPUDevice (rpu_transfer_device.cpp:679)
    "noise.key0",  "noise.key1",               // Philox key of all run-time noise
    "noise.forward_calls", "noise.backward_calls", "noise.update_calls", "noise.transfer_calls",
    "noise.weight_op_calls",
    "rpu_device.transfer_counter",             // ChoppedTransferRPUDevice (passes over the matrix)
    "rpu_device.mixed.current_update_index",   // MixedPrecRPUDeviceBase (rpu_mixedprec_device_base.cpp:252-253)
    "rpu_device.mixed.current_row_index",
};
constexpr int kExtraCount = (int)(sizeof(kExtraNames) / sizeof(kExtraNames[0]));
} // namespace

int Tile::extraCount() { return kExtraCount; }

const char *Tile::extraName(int k) {
  if (k < 0 || k >= kExtraCount) {
    AB200_FATAL("extra state index out of range");
  }
  return kExtraNames[k];
}

void Tile::dumpExtra(double *values) const {
  const double v[kExtraCount] = {(double)lr_,
                                 (double)update_idx_,
                                 (double)slice_idx_,
                                 (double)key_.k0,
                                 (double)key_.k1,
                                 (double)fwd_calls_,
                                 (double)bwd_calls_,
                                 (double)upd_calls_,
                                 (double)transfer_calls_,
                                 (double)op_calls_,
                                 (double)chop_passes_,
                                 (double)mp_update_idx_,
                                 (double)mp_row_idx_};
  for (int k = 0; k < kExtraCount; k++) {
    values[k] = v[k];
  }
}

void Tile::loadExtra(const char *const *names, const double *values, int n, bool strict) {
  bool seen[kExtraCount] = {};
  for (int e = 0; e < n; e++) {
    int k = 0;
    while (k < kExtraCount && std::strcmp(names[e], kExtraNames[k]) != 0) {
      k++;
    }
    if (k == kExtraCount) {
      if (strict) {
        AB200_FATAL("load_extra: unexpected key '" << names[e] << "'");
      }
      continue;
    }
    seen[k] = true;
    const double v = values[e];
    switch (k) {
    case 0: lr_ = (float)v; break;
    case 1: update_idx_ = (long long)v; break;
    case 2: slice_idx_ = (int)v; break;
    case 3: key_.k0 = (uint32_t)v; break;
    case 4: key_.k1 = (uint32_t)v; break;
    case 5: fwd_calls_ = (uint32_t)v; break;
    case 6: bwd_calls_ = (uint32_t)v; break;
    case 7: upd_calls_ = (uint32_t)v; break;
    case 8: transfer_calls_ = (uint32_t)v; break;
    case 9: op_calls_ = (uint32_t)v; break;
    case 10: chop_passes_ = (uint64_t)v; break;
    case 11: mp_update_idx_ = (long long)v; break;
    case 12: mp_row_idx_ = (int)v; break;
    }
  }
  if (strict) {
    for (int k = 0; k < kExtraCount; k++) {
      if (!seen[k]) {
        AB200_FATAL("load_extra: key '" << kExtraNames[k] << "' is missing"); // RPU::load, strict
      }
    }
  }
}

// Vector-valued state of the chopped / dynamic transfer compounds: the choppers of the input and
// output lines and, for the dynamic form, which input choppers flipped at their last transfer
// (in_chopper_, out_chopper_, in_chopper_switched_ of the reference's dumpExtra,
// rpu_chopped_transfer_device.cpp:229-262, rpu_dynamic_transfer_device.cpp:196-236).
int Tile::extraVectorCount() const {
  if (cfg_.device_kind != AB200_DEVICE_TRANSFER || !cfg_.transfer.chopped) {
    return 0;
  }
  return cfg_.transfer.dynamic ? 3 : 2;
}

const char *Tile::extraVectorName(int k) const {
  static const char *const kNames[3] = {"rpu_device.in_chopper", "rpu_device.out_chopper",
                                        "rpu_device.in_chopper_switched"};
  if (k < 0 || k >= extraVectorCount()) {
    AB200_FATAL("extra vector index out of range");
  }
  return kNames[k];
}

int Tile::extraVectorSize(int k) const {
  if (k < 0 || k >= extraVectorCount()) {
    AB200_FATAL("extra vector index out of range");
  }
  return k == 1 ? d_size_ : x_size_;
}

void Tile::getExtraVector(int k, double *out) {
  const int n = extraVectorSize(k);
  if (k == 2) {
    for (int i = 0; i < n; i++) {
      out[i] = i < (int)chop_switched_.size() ? (double)chop_switched_[i] : 0.0;
    }
    return;
  }
  if (device_ < 0) {
    std::fill(out, out + n, 0.0); // all choppers start unflipped
    return;
  }
  requireDevice("dump_extra");
  std::vector<unsigned char> t((size_t)n);
  AB200_CUDA(cudaDeviceSynchronize());
  AB200_CUDA(cudaMemcpy(t.data(), k == 0 ? chop_in_ : chop_out_, (size_t)n, cudaMemcpyDeviceToHost));
  for (int i = 0; i < n; i++) {
    out[i] = (double)t[i];
  }
}

void Tile::setExtraVector(int k, const double *in, int n) {
  if (n != extraVectorSize(k)) {
    AB200_FATAL("load_extra: '" << extraVectorName(k) << "' expects " << extraVectorSize(k) << " values");
  }
  if (k == 2) {
    chop_switched_.assign((size_t)n, 0);
    for (int i = 0; i < n; i++) {
      chop_switched_[i] = in[i] != 0.0 ? 1 : 0;
    }
    return;
  }
  requireDevice("load_extra");
  std::vector<unsigned char> t((size_t)n);
  for (int i = 0; i < n; i++) {
    t[i] = in[i] != 0.0 ? 1 : 0;
  }
  AB200_CUDA(cudaDeviceSynchronize());
  AB200_CUDA(cudaMemcpy(k == 0 ? chop_in_ : chop_out_, t.data(), (size_t)n, cudaMemcpyHostToDevice));
}

Tile::~Tile() {
  if (device_ >= 0) {
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(device_);
    cudaFree(w_owned_);
    cudaFree(w_fast_);
    for (int k = 0; k < 2; k++) {
      cudaFree(dev_[k].par4);
      cudaFree(dev_[k].par2);
      cudaFree(dev_[k].par3);
      cudaFree(dev_[k].pw);
    }
    cudaFree(scale_);
    cudaFree(factor_);
    cudaFree(vnorm_);
    cudaFree(sval_);
    cudaFree(flags_);
    cudaFree(bm_stats_);
    cudaFree(fb_w_);
    cudaFree(fb_amax_);
    cudaFree(drift_prev_);
    cudaFree(drift_w0_);
    cudaFree(drift_t_);
    cudaFree(drift_nu_);
    cudaFree(xls_);
    cudaFree(xlx_);
    cudaFree(xloff_);
    cudaFree(chop_in_);
    cudaFree(chop_out_);
    cudaFree(nm_state_);
    cudaFree(f_lt_.voff);
    cudaFree(f_lt_.nl);
    cudaFree(b_lt_.voff);
    cudaFree(b_lt_.nl);
    cudaFree(f_onv_);
    cudaFree(b_onv_);
    cudaFree(xw_);
    cudaFree(dw_);
    cudaFree(xwt_);
    cudaFree(xnzt_);
    cudaFree(onehot_);
    cudaFree(tread_);
    cudaFree(t_words_);
    cudaFree(t_buffer_);
    cudaFree(t_mean_);
    cudaFree(t_past_);
    cudaFree(idx_);
    cudaFree(pulses_up_);
    cudaFree(pulses_down_);
    cudaFree(chi_);
    cudaFree(mp_qx_);
    cudaFree(mp_qd_);
    cudaFree(mp_counts_);
    cudaFree(mp_onehot_);
    cudaFree(idx_t_);
    cudaFree(csr_off_);
    cudaFree(csr_pos_);
    cudaFree(cols_x_);
    cudaFree(cols_d_);
    cudaFree(stage_dev_);
    cudaFree(acc_block_);
    cudaFree(clip_stats_);
    cudaFreeHost(stage_pinned_);
    if (prev >= 0) {
      cudaSetDevice(prev);
    }
  }
}

void Tile::requireDevice(const char *what) const {
  if (device_ < 0) {
    AB200_FATAL(what << ": the analog tile has no CPU compute path; move it to a CUDA device first");
  }
  AB200_CUDA(cudaSetDevice(device_));
}

void Tile::uploadDeviceStore(DeviceStore &ds) {
  if (ds.kind == AB200_DEVICE_IDEAL) {
    return;
  }
  const size_t size = (size_t)x_size_ * d_size_;
  std::vector<float4> p4(size);
  std::vector<float2> p2(size);
  const float *wmax = &ds.host[0 * size], *wmin = &ds.host[1 * size], *sup = &ds.host[2 * size],
              *sdown = &ds.host[3 * size];
  const float *e0 = nullptr, *e1 = nullptr;
  if (ds.kind == AB200_DEVICE_LINEAR_STEP || ds.kind == AB200_DEVICE_SOFT_BOUNDS ||
      ds.kind == AB200_DEVICE_POW_STEP) {
    e0 = &ds.host[8 * size];
    e1 = &ds.host[9 * size];
  } else if (ds.kind == AB200_DEVICE_SOFT_BOUNDS_REFERENCE) {
    e0 = &ds.host[8 * size];
  }
  for (int i = 0; i < d_size_; i++) {
    for (int j = 0; j < x_size_; j++) {
      size_t src = (size_t)i * x_size_ + j, dst = (size_t)j * d_size_ + i;
      p4[dst] = make_float4(sup[src], sdown[src], wmax[src], wmin[src]);
      p2[dst] = make_float2(e0 ? e0[src] : 0.0f, e1 ? e1[src] : 0.0f);
    }
  }
  if (!ds.par4) {
    AB200_CUDA(cudaMalloc(&ds.par4, size * sizeof(float4)));
    AB200_CUDA(cudaMalloc(&ds.par2, size * sizeof(float2)));
  }
  AB200_CUDA(cudaMemcpy(ds.par4, p4.data(), size * sizeof(float4), cudaMemcpyHostToDevice));
  AB200_CUDA(cudaMemcpy(ds.par2, p2.data(), size * sizeof(float2), cudaMemcpyHostToDevice));
  if (ds.kind == AB200_DEVICE_PIECEWISE_STEP) {
    if (!ds.pw) {
      AB200_CUDA(cudaMalloc(&ds.pw, ds.pw_host.size() * sizeof(float)));
    }
    AB200_CUDA(cudaMemcpy(ds.pw, ds.pw_host.data(), ds.pw_host.size() * sizeof(float),
                          cudaMemcpyHostToDevice));
  }
}

void Tile::toDevice(int cuda_device) {
  if (device_ >= 0) {
    if (device_ == cuda_device) {
      return;
    }
    AB200_FATAL("tile already lives on CUDA device " << device_);
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || cuda_device >= count) {
    AB200_FATAL("CUDA device " << cuda_device << " is not available ("
                               << (e != cudaSuccess ? cudaGetErrorString(e) : "index out of range")
                               << "); the analog tile has no CPU fallback");
  }
  AB200_CUDA(cudaSetDevice(cuda_device));
  device_ = cuda_device;
  const size_t size = (size_t)x_size_ * d_size_;
  AB200_CUDA(cudaMalloc(&w_owned_, size * sizeof(float)));
  w_ = w_owned_;
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    AB200_CUDA(cudaMalloc(&w_fast_, size * sizeof(float)));
    AB200_CUDA(cudaMemset(w_fast_, 0, size * sizeof(float)));
    AB200_CUDA(cudaMalloc(&onehot_, (size_t)x_size_ * sizeof(float)));
    AB200_CUDA(cudaMalloc(&tread_, (size_t)d_size_ * sizeof(float)));
    {
      // pulse words of the single sample of a transfer write (all its segments)
      const size_t nseg_t = (size_t)std::max(1, (cfg_.transfer.transfer_up.desired_bl + kPulseSegSlots - 1) /
                                                    kPulseSegSlots);
      AB200_CUDA(cudaMalloc(&t_words_, nseg_t * (size_t)(x_size_ + d_size_) * sizeof(uint32_t)));
    }
    if (cfg_.transfer.buffered) {
      AB200_CUDA(cudaMalloc(&t_buffer_, size * sizeof(float)));
      AB200_CUDA(cudaMemset(t_buffer_, 0, size * sizeof(float)));
    }
    if (cfg_.transfer.chopped) {
      // all choppers start unflipped (ChoppedTransferRPUDevice::populate,
      // rpu_chopped_transfer_device.cpp:214-227)
      AB200_CUDA(cudaMalloc(&chop_in_, (size_t)x_size_));
      AB200_CUDA(cudaMalloc(&chop_out_, (size_t)d_size_));
      AB200_CUDA(cudaMemset(chop_in_, 0, (size_t)x_size_));
      AB200_CUDA(cudaMemset(chop_out_, 0, (size_t)d_size_));
      chop_passes_ = 0;
    }
    if (cfg_.transfer.dynamic) {
      AB200_CUDA(cudaMalloc(&t_mean_, size * sizeof(float)));
      AB200_CUDA(cudaMalloc(&t_past_, size * sizeof(float)));
      AB200_CUDA(cudaMemset(t_mean_, 0, size * sizeof(float)));
      AB200_CUDA(cudaMemset(t_past_, 0, size * sizeof(float)));
      chop_switched_.assign((size_t)x_size_, 0);
    }
  }
  if (countsPulses()) {
    AB200_CUDA(cudaMalloc(&pulses_up_, size * sizeof(unsigned long long)));
    AB200_CUDA(cudaMalloc(&pulses_down_, size * sizeof(unsigned long long)));
    AB200_CUDA(cudaMemset(pulses_up_, 0, size * sizeof(unsigned long long)));
    AB200_CUDA(cudaMemset(pulses_down_, 0, size * sizeof(unsigned long long)));
  }
  if (cfg_.mixed.enabled) {
    AB200_CUDA(cudaMalloc(&chi_, size * sizeof(float)));
    AB200_CUDA(cudaMemset(chi_, 0, size * sizeof(float)));
    mp_update_idx_ = 0;
    mp_row_idx_ = 0;
    // the device's granularity unless set (MixedPrecRPUDeviceBase::populate,
    // rpu_mixedprec_device_base.cpp:229-240)
    mp_granularity_ = cfg_.mixed.granularity > 0.0f ? cfg_.mixed.granularity : dev_[0].dw_min;
    if (!(mp_granularity_ > 0.0f)) {
      AB200_FATAL("Cannot establish granularity from device. Need explicit setting >=0.");
    }
  }
  AB200_CUDA(cudaMalloc(&bm_stats_, 2 * sizeof(int)));
  AB200_CUDA(cudaMemset(bm_stats_, 0, 2 * sizeof(int)));
  {
    const float not_started = -1.0f; // aux_nm_value_ (rpu_forward_backward_pass.h:241)
    AB200_CUDA(cudaMalloc(&nm_state_, sizeof(float)));
    AB200_CUDA(cudaMemcpy(nm_state_, &not_started, sizeof(float), cudaMemcpyHostToDevice));
  }
  populateLineTables();
  for (int k = 0; k < n_dev_; k++) {
    uploadDeviceStore(dev_[k]);
  }
  std::vector<float> w = host_w_dx_;
  setWeights(w.data());
  host_w_dx_.clear();
  host_w_dx_.shrink_to_fit();
}

// Per-line values of the two IO directions (ForwardBackwardPassIOManaged::populateFBParameter,
// rpu_forward_backward_pass.cpp:249-316): voltage offsets, output non-linearities with the slope
// calibration factor, output-noise values. Drawn on the host from the tile's seed.
static bool ioHasVOffset(const IOEff &io) {
  return !io.is_perfect && (io.v_offset_std > 0.0f || io.r_series > 0.0f);
}
static bool ioHasNl(const IOEff &io) {
  return !io.is_perfect && (io.out_nl > 0.0f || io.r_series > 0.0f);
}
static float nlFactor(const IOEff &io, const std::vector<float> &nl) {
  if (!(io.slope_calibration > 0.0f)) {
    return 1.0f;
  }
  const float out_bound = (io.out_bound > 0.0f && io.out_bound < std::numeric_limits<float>::infinity())
                              ? io.out_bound
                              : 1.0f;
  float sum = 0.0f;
  if (io.out_nl > 0.0f || !nl.empty()) {
    for (float v : nl) {
      sum += std::fabs(v);
    }
  }
  const float n = nl.empty() ? 1.0f : (float)nl.size();
  const float f = 1.0f + (sum / n + io.r_series) * io.slope_calibration * out_bound;
  return f * f;
}

void Tile::uploadLineTables(LineTables &lt, const IOEff &io, int n, float **onv) {
  auto up = [&](const std::vector<float> &h, float **dst) {
    if (h.empty()) {
      return;
    }
    if (!*dst) {
      AB200_CUDA(cudaMalloc(dst, h.size() * sizeof(float)));
    }
    AB200_CUDA(cudaMemcpy(*dst, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice));
  };
  (void)n;
  up(lt.h_voff, &lt.voff);
  up(lt.h_nl, &lt.nl);
  up(lt.h_onv, onv);
  lt.nl_factor = ioHasNl(io) ? nlFactor(io, lt.h_nl) : 1.0f;
}

void Tile::populateLineTables() {
  HostRNG rng(key_.k0 ^ (key_.k1 * 0x9e3779b9u) ^ 0x6f6e7631u);
  auto draw = [&](const IOEff &io, int n, LineTables &lt, float **onv) {
    if (io.is_perfect) {
      return;
    }
    if (ioHasVOffset(io)) {
      lt.h_voff.resize((size_t)n);
      for (auto &e : lt.h_voff) {
        e = std::max(io.v_offset_std * rng.gauss(), 0.0f);
      }
    }
    if (ioHasNl(io)) {
      const float out_bound =
          (io.out_bound > 0.0f && io.out_bound < std::numeric_limits<float>::infinity()) ? io.out_bound : 1.0f;
      lt.h_nl.resize((size_t)n);
      for (auto &e : lt.h_nl) {
        e = std::fabs(io.out_nl / out_bound * (1.0f + std::max(io.out_nl_std, 0.0f) * rng.gauss()));
      }
    }
    if (io.out_noise_std > 0.0f) {
      lt.h_onv.resize((size_t)n);
      for (auto &e : lt.h_onv) {
        e = std::fabs(io.out_noise * (1.0f + io.out_noise_std * rng.gauss()));
      }
    }
    uploadLineTables(lt, io, n, onv);
  };
  draw(f_io_, d_size_, f_lt_, &f_onv_);
  draw(b_io_, x_size_, b_lt_, &b_onv_);
}

void Tile::setLineTables(MvmProblem &p, const LineTables &lt, const float *onv) const {
  p.out_noise_vals = onv;
  p.v_offset = lt.voff;
  p.out_nl = lt.nl;
  p.nl_factor = lt.nl_factor;
}

void Tile::getIoVector(bool backward, int which, float *values, int n) {
  const LineTables &lt = backward ? b_lt_ : f_lt_;
  const std::vector<float> &h = which == AB200_IOVEC_V_OFFSET
                                    ? lt.h_voff
                                    : (which == AB200_IOVEC_OUT_NONLINEARITY ? lt.h_nl : lt.h_onv);
  if (which < AB200_IOVEC_V_OFFSET || which > AB200_IOVEC_OUT_NOISE_VALUES) {
    AB200_FATAL("io vector: unknown kind");
  }
  if (h.empty()) {
    AB200_FATAL("io vector: the IO setting that uses it is off for this direction");
  }
  if (n != (int)h.size()) {
    AB200_FATAL("io vector: expected " << h.size() << " values");
  }
  std::memcpy(values, h.data(), h.size() * sizeof(float));
}

void Tile::setIoVector(bool backward, int which, const float *values, int n) {
  requireDevice("set_io_vector");
  LineTables &lt = backward ? b_lt_ : f_lt_;
  if (which < AB200_IOVEC_V_OFFSET || which > AB200_IOVEC_OUT_NOISE_VALUES) {
    AB200_FATAL("io vector: unknown kind");
  }
  std::vector<float> &h = which == AB200_IOVEC_V_OFFSET
                              ? lt.h_voff
                              : (which == AB200_IOVEC_OUT_NONLINEARITY ? lt.h_nl : lt.h_onv);
  if (h.empty()) {
    AB200_FATAL("io vector: the IO setting that uses it is off for this direction");
  }
  if (n != (int)h.size()) {
    AB200_FATAL("io vector: expected " << h.size() << " values");
  }
  AB200_CUDA(cudaDeviceSynchronize());
  h.assign(values, values + n);
  uploadLineTables(lt, backward ? b_io_ : f_io_, n, backward ? &b_onv_ : &f_onv_);
}

void Tile::ensureScratch(int m) {
  if (m <= scratch_m_) {
    return;
  }
  AB200_CUDA(cudaDeviceSynchronize());
  cudaFree(scale_);
  cudaFree(factor_);
  cudaFree(vnorm_);
  cudaFree(sval_);
  cudaFree(flags_);
  cudaFree(xw_);
  cudaFree(dw_);
  int cap = m + m / 4 + 16;
  AB200_CUDA(cudaMalloc(&scale_, (size_t)cap * sizeof(float)));
  AB200_CUDA(cudaMalloc(&factor_, (size_t)cap * sizeof(float)));
  AB200_CUDA(cudaMalloc(&vnorm_, (size_t)cap * sizeof(float)));
  AB200_CUDA(cudaMalloc(&sval_, (size_t)cap * sizeof(float)));
  AB200_CUDA(cudaMalloc(&flags_, (size_t)cap * sizeof(int)));
  // the flags are zero between passes: a pass sets them, the re-run clears the ones it serves
  AB200_CUDA(cudaMemset(flags_, 0, (size_t)cap * sizeof(int)));
  xw_ = dw_ = nullptr;
  if (cfg_.device_kind != AB200_DEVICE_IDEAL && up_.pulse_type != AB200_PULSE_NONE) {
    AB200_CUDA(cudaMalloc(&xw_, (size_t)cap * x_size_ * sizeof(uint32_t)));
    AB200_CUDA(cudaMalloc(&dw_, (size_t)cap * d_size_ * sizeof(uint32_t)));
  }
  scratch_m_ = cap;
}

void Tile::ensureStreamScratch(int m_pad) {
  const size_t need = (size_t)m_pad * x_size_;
  if (need <= xwt_words_) {
    return;
  }
  AB200_CUDA(cudaDeviceSynchronize());
  cudaFree(xwt_);
  cudaFree(xnzt_);
  cudaFree(xls_);
  cudaFree(xlx_);
  cudaFree(xloff_);
  xwt_ = xnzt_ = xls_ = xlx_ = xloff_ = nullptr;
  const size_t cap = need + need / 8;
  AB200_CUDA(cudaMalloc(&xwt_, cap * sizeof(uint32_t)));
  AB200_CUDA(cudaMalloc(&xnzt_, (cap / 32 + x_size_) * sizeof(uint32_t)));
  AB200_CUDA(cudaMalloc(&xls_, cap * sizeof(uint32_t)));
  AB200_CUDA(cudaMalloc(&xlx_, cap * sizeof(uint32_t)));
  AB200_CUDA(cudaMalloc(&xloff_, (cap / 32 + 2 * (size_t)x_size_) * sizeof(uint32_t)));
  xwt_words_ = cap;
}

void Tile::ensureStage(size_t n_floats) {
  if (n_floats <= stage_floats_) {
    return;
  }
  AB200_CUDA(cudaDeviceSynchronize());
  cudaFree(stage_dev_);
  cudaFreeHost(stage_pinned_);
  AB200_CUDA(cudaMalloc(&stage_dev_, n_floats * sizeof(float)));
  AB200_CUDA(cudaMallocHost(&stage_pinned_, n_floats * sizeof(float)));
  stage_floats_ = n_floats;
}

// ---------------------------------------------------------------------------------------------
// weights
// ---------------------------------------------------------------------------------------------
void Tile::setWeights(const float *w_host_dx) {
  const size_t size = (size_t)x_size_ * d_size_;
  if (device_ < 0) {
    // host carrier: clip to the (slow / only) device's bounds like onSetWeights
    host_w_dx_.assign(w_host_dx, w_host_dx + size);
    const DeviceStore &ds = dev_[n_dev_ - 1];
    if (ds.kind != AB200_DEVICE_IDEAL) {
      for (size_t k = 0; k < size; k++) {
        host_w_dx_[k] = std::max(std::min(host_w_dx_[k], ds.host[k]), ds.host[size + k]);
      }
    }
    return;
  }
  requireDevice("set_weights");
  std::vector<float> t(size);
  for (int i = 0; i < d_size_; i++) {
    for (int j = 0; j < x_size_; j++) {
      t[(size_t)j * d_size_ + i] = w_host_dx[(size_t)i * x_size_ + j];
    }
  }
  AB200_CUDA(cudaMemcpy(w_, t.data(), size * sizeof(float), cudaMemcpyHostToDevice));
  setWeightsDevice(nullptr, nullptr);
}

void Tile::setWeightsDevice(const float *w_dev_xd, cudaStream_t s) {
  requireDevice("set_weights");
  const size_t size = (size_t)x_size_ * d_size_;
  if (w_dev_xd && w_dev_xd != w_) {
    AB200_CUDA(cudaMemcpyAsync(w_, w_dev_xd, size * sizeof(float), cudaMemcpyDeviceToDevice, s));
  }
  // RPUPulsed::setWeights -> onSetWeights (rpu_pulsed.cpp:288-292): clip to device bounds;
  // Transfer additionally zeroes the fast tile and resets its counters
  // (rpu_transfer_device.cpp:559-602).
  DeviceStore &ds = dev_[n_dev_ - 1];
  if (ds.kind != AB200_DEVICE_IDEAL) {
    launchClipToBounds(w_, ds.par4, (long long)size, s);
  }
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    AB200_CUDA(cudaMemsetAsync(w_fast_, 0, size * sizeof(float), s));
    update_idx_ = 0;
    slice_idx_ = 0;
  }
  if (cfg_.mixed.enabled) {
    // MixedPrecRPUDevice::onSetWeights (rpu_mixedprec_device.cpp:348-355): chi and the counters start again
    AB200_CUDA(cudaMemsetAsync(chi_, 0, size * sizeof(float), s));
    mp_update_idx_ = 0;
    mp_row_idx_ = 0;
  }
  w_version_++;
  AB200_CUDA(cudaStreamSynchronize(s));
}

void Tile::getWeights(float *w_host_dx) {
  const size_t size = (size_t)x_size_ * d_size_;
  if (device_ < 0) {
    std::memcpy(w_host_dx, host_w_dx_.data(), size * sizeof(float));
    return;
  }
  requireDevice("get_weights");
  std::vector<float> t(size);
  AB200_CUDA(cudaDeviceSynchronize());
  AB200_CUDA(cudaMemcpy(t.data(), w_, size * sizeof(float), cudaMemcpyDeviceToHost));
  for (int i = 0; i < d_size_; i++) {
    for (int j = 0; j < x_size_; j++) {
      w_host_dx[(size_t)i * x_size_ + j] = t[(size_t)j * d_size_ + i];
    }
  }
}

void Tile::getWeightsDevice(float *w_dev_xd, cudaStream_t s) {
  requireDevice("get_weights");
  AB200_CUDA(cudaMemcpyAsync(w_dev_xd, w_, (size_t)x_size_ * d_size_ * sizeof(float),
                             cudaMemcpyDeviceToDevice, s));
}

void Tile::setSharedWeights(float *w_dev_xd, uint64_t version) {
  requireDevice("set_shared_weights");
  if (!w_dev_xd) {
    AB200_FATAL("set_shared_weights: null pointer");
  }
  if (w_ != w_dev_xd || shared_version_ != version) {
    w_version_++;
  }
  w_ = w_dev_xd;
  shared_version_ = version;
}

void Tile::setDeltaWeights(float *dw_dev_xd) {
  if (dw_dev_xd) {
    requireDevice("set_delta_weights");
  }
  delta_w_ = dw_dev_xd;
}

// ---------------------------------------------------------------------------------------------
// hidden parameters: [name][d][x], names as the reference reports them
// (PulsedRPUDevice::getDPNames rpu_pulsed_device.cpp:235-253; VectorRPUDevice :188-203)
// ---------------------------------------------------------------------------------------------
int Tile::hiddenCount() const {
  if (cfg_.device_kind == AB200_DEVICE_IDEAL) {
    return 0;
  }
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
    return (int)dev_[0].names.size() + (int)dev_[1].names.size() + 2 +
           (cfg_.transfer.dynamic ? 3 : cfg_.transfer.buffered ? 1 : 0);
  }
  return (int)dev_[0].names.size() + (cfg_.mixed.enabled ? 1 : 0);
}

const char *Tile::hiddenName(int i) const {
  static thread_local std::string buf;
  if (i < 0 || i >= hiddenCount()) {
    return "";
  }
  if (cfg_.device_kind != AB200_DEVICE_TRANSFER) {
    if (i == (int)dev_[0].names.size()) {
      return "hidden_weights_chi"; // MixedPrecRPUDeviceBase::getDPNames (rpu_mixedprec_device_base.cpp:368-378)
    }
    return dev_[0].names[i].c_str();
  }
  int n0 = (int)dev_[0].names.size();
  if (cfg_.transfer.dynamic && i >= hiddenCount() - 3) {
    // rpu_dynamic_transfer_device.cpp:361-382
    static const char *const kDynamic[3] = {"buffered_FP_weight", "running_mean_weight", "past_mean_weight"};
    return kDynamic[i - (hiddenCount() - 3)];
  }
  if (cfg_.transfer.buffered && i == hiddenCount() - 1) {
    buf = "buffered_FP_weight_0"; // rpu_buffered_transfer_device.cpp:217-227
    return buf.c_str();
  }
  int k = i <= n0 ? 0 : 1;
  int local = k == 0 ? i : i - n0 - 1;
  int nk = (int)dev_[k].names.size();
  buf = local < nk ? dev_[k].names[local] + "_" + std::to_string(k)
                   : "hidden_weights_" + std::to_string(k);
  return buf.c_str();
}

void Tile::getHidden(float *out) {
  const size_t size = (size_t)x_size_ * d_size_;
  if (cfg_.device_kind == AB200_DEVICE_IDEAL) {
    return;
  }
  if (cfg_.device_kind != AB200_DEVICE_TRANSFER) {
    std::memcpy(out, dev_[0].host.data(), dev_[0].host.size() * sizeof(float));
    if (cfg_.mixed.enabled) {
      float *o = out + dev_[0].host.size();
      if (device_ >= 0) {
        std::vector<float> t(size);
        AB200_CUDA(cudaDeviceSynchronize());
        AB200_CUDA(cudaMemcpy(t.data(), chi_, size * sizeof(float), cudaMemcpyDeviceToHost));
        for (int i = 0; i < d_size_; i++) {
          for (int j = 0; j < x_size_; j++) {
            o[(size_t)i * x_size_ + j] = t[(size_t)j * d_size_ + i];
          }
        }
      } else {
        std::memset(o, 0, size * sizeof(float));
      }
    }
    return;
  }
  float *o = out;
  for (int k = 0; k < 2; k++) {
    std::memcpy(o, dev_[k].host.data(), dev_[k].host.size() * sizeof(float));
    o += dev_[k].host.size();
    // hidden weights of device k: fast tile A for k = 0, the visible weights for k = 1
    if (device_ >= 0) {
      requireDevice("get_hidden_parameters");
      std::vector<float> t(size);
      AB200_CUDA(cudaDeviceSynchronize());
      AB200_CUDA(cudaMemcpy(t.data(), k == 0 ? w_fast_ : w_, size * sizeof(float),
                            cudaMemcpyDeviceToHost));
      for (int i = 0; i < d_size_; i++) {
        for (int j = 0; j < x_size_; j++) {
          o[(size_t)i * x_size_ + j] = t[(size_t)j * d_size_ + i];
        }
      }
    } else if (k == 1) {
      std::memcpy(o, host_w_dx_.data(), size * sizeof(float));
    } else {
      std::memset(o, 0, size * sizeof(float));
    }
    o += size;
  }
  // digital planes of the buffered forms: the buffer, then (dynamic) running and reference mean
  const float *planes[3] = {t_buffer_, t_mean_, t_past_};
  const int n_planes = cfg_.transfer.dynamic ? 3 : cfg_.transfer.buffered ? 1 : 0;
  for (int q = 0; q < n_planes; q++) {
    if (device_ >= 0) {
      std::vector<float> t(size);
      AB200_CUDA(cudaMemcpy(t.data(), planes[q], size * sizeof(float), cudaMemcpyDeviceToHost));
      for (int i = 0; i < d_size_; i++) {
        for (int j = 0; j < x_size_; j++) {
          o[(size_t)i * x_size_ + j] = t[(size_t)j * d_size_ + i];
        }
      }
    } else {
      std::memset(o, 0, size * sizeof(float));
    }
    o += size;
  }
}

void Tile::setHidden(const float *in) {
  const size_t size = (size_t)x_size_ * d_size_;
  if (cfg_.device_kind == AB200_DEVICE_IDEAL) {
    return;
  }
  const float *p = in;
  if (drift_prev_ && device_ >= 0) {
    // new drift exponents: the drift state starts again with the next drift call
    AB200_CUDA(cudaDeviceSynchronize());
    cudaFree(drift_prev_);
    cudaFree(drift_w0_);
    cudaFree(drift_t_);
    cudaFree(drift_nu_);
    drift_prev_ = drift_w0_ = drift_t_ = drift_nu_ = nullptr;
  }
  for (int k = 0; k < n_dev_; k++) {
    std::memcpy(dev_[k].host.data(), p, dev_[k].host.size() * sizeof(float));
    dev_[k].par3_valid = false;
    p += dev_[k].host.size();
    // PulsedRPUDevice::setDeviceParameter re-estimates dw_min from the given step sizes when it
    // moved by more than 2 * dw_min_dtod (rpu_pulsed_device.cpp:319-334)
    const float *sup = &dev_[k].host[2 * size], *sdown = &dev_[k].host[3 * size];
    double acc = 0.0;
    for (size_t e = 0; e < size; e++) {
      acc += (fabsf(sup[e]) + fabsf(sdown[e])) / 2.0f;
    }
    float est = (float)(acc / (double)size);
    if (fabsf(est - cfg_.device[k].dw_min) / cfg_.device[k].dw_min > 2.0f * cfg_.device[k].dw_min_dtod) {
      cfg_.device[k].dw_min = est; // the parameter itself, then the granularity derived from it
      dev_[k].dw_min = weightGranularity(cfg_.device[k], dev_[k].kind);
    }
    if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
      if (device_ >= 0 && k == 0) {
        requireDevice("set_hidden_parameters");
        std::vector<float> t(size);
        for (int i = 0; i < d_size_; i++) {
          for (int j = 0; j < x_size_; j++) {
            t[(size_t)j * d_size_ + i] = p[(size_t)i * x_size_ + j];
          }
        }
        AB200_CUDA(cudaMemcpy(w_fast_, t.data(), size * sizeof(float), cudaMemcpyHostToDevice));
      }
      p += size;
    }
    if (device_ >= 0) {
      requireDevice("set_hidden_parameters");
      uploadDeviceStore(dev_[k]);
    }
  }
  if (cfg_.mixed.enabled && device_ >= 0) {
    std::vector<float> t(size);
    for (int i = 0; i < d_size_; i++) {
      for (int j = 0; j < x_size_; j++) {
        t[(size_t)j * d_size_ + i] = p[(size_t)i * x_size_ + j];
      }
    }
    AB200_CUDA(cudaMemcpy(chi_, t.data(), size * sizeof(float), cudaMemcpyHostToDevice));
  }
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER && cfg_.transfer.buffered && device_ >= 0) {
    float *planes[3] = {t_buffer_, t_mean_, t_past_};
    const int n_planes = cfg_.transfer.dynamic ? 3 : 1;
    std::vector<float> t(size);
    for (int q = 0; q < n_planes; q++) {
      for (int i = 0; i < d_size_; i++) {
        for (int j = 0; j < x_size_; j++) {
          t[(size_t)j * d_size_ + i] = p[(size_t)i * x_size_ + j];
        }
      }
      AB200_CUDA(cudaMemcpy(planes[q], t.data(), size * sizeof(float), cudaMemcpyHostToDevice));
      p += size;
    }
  }
  // weights are re-clipped to the new bounds (onSetWeights at the end of setDeviceParameter)
  w_version_++;
  if (device_ >= 0) {
    launchClipToBounds(w_, dev_[n_dev_ - 1].par4, (long long)size, nullptr);
    if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
      launchClipToBounds(w_fast_, dev_[0].par4, (long long)size, nullptr);
    }
    AB200_CUDA(cudaDeviceSynchronize());
  } else {
    std::vector<float> w = host_w_dx_;
    setWeights(w.data());
  }
}

// ---------------------------------------------------------------------------------------------
// forward / backward
// ---------------------------------------------------------------------------------------------
void Tile::fillMvmScratch(MvmProblem &p) {
  ensureScratch(p.m);
  p.scale = scale_;
  p.factor = factor_;
  p.vnorm = vnorm_;
  p.sval = sval_;
  p.flags = flags_;
  p.bm_stats = bm_stats_;
  p.nm_state = nm_state_;
  p.key = key_;
}

void Tile::forward(const float *x, float *d, bool bias, int m, bool x_trans, bool d_trans,
                   bool is_test, cudaStream_t s, int out_t_rows) {
  // the IO noise is present in test mode too (rpu_forward_backward_pass.cpp:808-810); is_test only
  // selects between the weights and their modified copy
  requireDevice("forward");
  if (m <= 0) {
    return;
  }
  MvmProblem p{};
  p.in = x;
  const int x_in = x_size_ - (bias ? 1 : 0);
  p.in_ss = x_trans ? 1 : x_in;
  p.in_fs = x_trans ? m : 1;
  p.in_size = x_size_;
  p.in_real = x_in;
  p.out = d;
  // a transposed output [d_size][m] is the transposed store with one block of m rows, which the
  // tensor-core kernels write too
  if (d_trans && out_t_rows == 0) {
    out_t_rows = m;
    d_trans = false;
  }
  p.out_ss = d_trans ? 1 : d_size_;
  p.out_fs = d_trans ? m : 1;
  p.out_size = d_size_;
  p.out_store = d_size_;
  p.accumulate = 0;
  p.w = fbWeights(is_test);
  p.wk = d_size_;
  p.wn = 1;
  p.m = m;
  p.backward = 0;
  p.io = f_io_;
  setLineTables(p, f_lt_, f_onv_);
  p.alpha = 1.0f;
  p.call = fwd_calls_++;
  p.noise_id = 0;
  p.out_t_rows = out_t_rows;
  fillMvmScratch(p);
  if (tcEligible(p)) {
    AB200_CUDA(cudaMemsetAsync(bm_stats_, 0, 2 * sizeof(int), s));
    runTc(p, s);
    launchBmRerun(p, s);
  } else {
    launchMvm(p, s); // its first kernel zeroes the re-run counters
  }
}

// Forward pass over rows that the DAC kernel gathers from whole images (indexed convolution
// interface): the tensor-core path of forward() with the unfolded matrix left out.
bool Tile::forwardGatherEligible(int b) const {
  static const bool off = [] {
    const char *e = getenv("AB200_INDEXED_GATHER");
    return e && e[0] == '0';
  }();
  MvmProblem p{};
  p.in_fs = p.out_fs = 1;
  p.in_size = p.in_real = x_size_;
  p.out_size = p.out_store = d_size_;
  p.m = b;
  p.io = f_io_;
  setLineTables(p, f_lt_, f_onv_);
  return !off && tcEligible(p) && TcEngine::gatherSupported(x_size_);
}

void Tile::forwardGathered(const float *images, const RowGather &g, float *d, int b, bool is_test,
                           cudaStream_t s, int out_t_rows) {
  MvmProblem p{};
  p.in = images;
  p.gather = g;
  p.out_t_rows = out_t_rows;
  p.in_ss = x_size_;
  p.in_fs = 1;
  p.in_size = x_size_;
  p.in_real = x_size_;
  p.out = d;
  p.out_ss = d_size_;
  p.out_fs = 1;
  p.out_size = d_size_;
  p.out_store = d_size_;
  p.accumulate = 0;
  p.w = fbWeights(is_test);
  p.wk = d_size_;
  p.wn = 1;
  p.m = b;
  p.backward = 0;
  p.io = f_io_;
  setLineTables(p, f_lt_, f_onv_);
  p.alpha = 1.0f;
  p.call = fwd_calls_++;
  p.noise_id = 0;
  fillMvmScratch(p);
  AB200_CUDA(cudaMemsetAsync(bm_stats_, 0, 2 * sizeof(int), s));
  runTc(p, s);
  launchBmRerun(p, s);
}

void Tile::forwardStrided(const float *x, long long x_ss, float *y, long long y_ss, int m,
                          bool accumulate, uint32_t noise_id, float out_scale, cudaStream_t s) {
  requireDevice("forward");
  MvmProblem p{};
  p.in = x;
  p.in_ss = x_ss;
  p.in_fs = 1;
  p.in_size = x_size_;
  p.in_real = x_size_;
  p.out = y;
  p.out_ss = y_ss;
  p.out_fs = 1;
  p.out_size = d_size_;
  p.out_store = d_size_;
  p.accumulate = accumulate ? 1 : 0;
  p.w = fbWeights(true);
  p.wk = d_size_;
  p.wn = 1;
  p.m = m;
  p.backward = 0;
  p.io = f_io_;
  setLineTables(p, f_lt_, f_onv_);
  p.alpha = out_scale; // digital scale of this tile's output (mapping scale)
  p.call = fwd_calls_++;
  p.noise_id = noise_id;
  fillMvmScratch(p);
  // The bound-management re-run rewrites whole output rows, so a tile that adds to the sum of
  // the earlier in-splits computes into its own block first and is added afterwards.
  const bool bm = !f_io_.is_perfect && f_io_.bm != AB200_BM_NONE;
  const bool via_block = accumulate && bm;
  if (via_block) {
    const size_t need = (size_t)m * d_size_;
    if (need > acc_block_floats_) {
      AB200_CUDA(cudaStreamSynchronize(s));
      cudaFree(acc_block_);
      acc_block_ = nullptr;
      AB200_CUDA(cudaMalloc(&acc_block_, need * sizeof(float)));
      acc_block_floats_ = need;
    }
    p.out = acc_block_;
    p.out_ss = d_size_;
    p.accumulate = 0;
  }
  if (!p.accumulate && tcEligible(p)) {
    AB200_CUDA(cudaMemsetAsync(bm_stats_, 0, 2 * sizeof(int), s));
    runTc(p, s);
    launchBmRerun(p, s);
  } else {
    launchMvm(p, s); // its first kernel zeroes the re-run counters
  }
  if (via_block) {
    launchAddBlock(acc_block_, d_size_, y, y_ss, m, d_size_, s);
  }
}

void Tile::backward(const float *d, float *x, bool bias, int m, bool d_trans, bool x_trans,
                    cudaStream_t s) {
  const int x_out = x_size_ - (bias ? 1 : 0);
  if (x_trans && !bias) {
    // transposed output [x_size][m]: the transposed store with one block of m rows
    backwardCore(d, d_trans ? 1 : d_size_, d_trans ? m : 1, x, x_size_, 1, x_out, m, false, 0, 1.0f, s, m);
    return;
  }
  backwardCore(d, d_trans ? 1 : d_size_, d_trans ? m : 1, x, x_trans ? 1 : x_out, x_trans ? m : 1,
               x_out, m, false, 0, 1.0f, s);
}

// used by the mapped array: backward on sub-blocks of wider gradient matrices
void Tile::backwardStrided(const float *d, long long d_ss, float *x, long long x_ss, int m,
                           bool accumulate, uint32_t noise_id, float out_scale, cudaStream_t s) {
  backwardCore(d, d_ss, 1, x, x_ss, 1, x_size_, m, accumulate, noise_id, out_scale, s);
}

void Tile::backwardCore(const float *d, long long d_ss, long long d_fs, float *x, long long x_ss,
                        long long x_fs, int x_store, int m, bool accumulate, uint32_t noise_id,
                        float out_scale, cudaStream_t s, int out_t_rows) {
  requireDevice("backward");
  if (m <= 0) {
    return;
  }
  MvmProblem p{};
  p.in = d;
  p.in_ss = d_ss;
  p.in_fs = d_fs;
  p.in_size = d_size_;
  p.in_real = d_size_;
  p.out = x;
  p.out_ss = x_ss;
  p.out_fs = x_fs;
  p.out_size = x_size_;
  p.out_store = x_store; // a bias column is computed but not returned (rpu.cpp:670-690)
  p.accumulate = accumulate ? 1 : 0;
  p.w = fbWeights(false);
  p.wk = 1; // W(k = d, n = x) = w[x * d_size + d]
  p.wn = d_size_;
  p.m = m;
  p.backward = 1;
  p.io = b_io_;
  setLineTables(p, b_lt_, b_onv_);
  p.alpha = out_scale;
  p.call = bwd_calls_++;
  p.noise_id = noise_id;
  p.out_t_rows = out_t_rows;
  fillMvmScratch(p);
  if (!accumulate && tcEligible(p)) {
    runTc(p, s);
  } else {
    launchMvm(p, s);
  }
}

// Tensor-core path: rows contiguous, no bias column, DAC codes representable, and either forced
// or large enough that the extra kernels (operand split, DAC) pay off.
bool Tile::tcEligible(const MvmProblem &p) const {
  const int mode = mvmPath();
  if (mode == 1) {
    return false;
  }
  if (p.in_fs != 1 || p.out_fs != 1 || p.in_real != p.in_size || p.out_store != p.out_size ||
      !TcEngine::ioSupported(p.io, p.out_noise_vals != nullptr)) {
    return false;
  }
  if (mode >= 2) {
    return true;
  }
  return p.m >= 128 && (double)p.m * p.in_size * p.out_size >= 16777216.0;
}

void Tile::runTc(const MvmProblem &p, cudaStream_t s) {
  std::unique_ptr<TcEngine> &eng = p.backward ? tc_bwd_ : tc_fwd_;
  uint64_t &ver = p.backward ? tc_bwd_version_ : tc_fwd_version_;
  if (!eng) {
    eng.reset(new TcEngine(device_));
    eng->configure({p.in_size}, {p.out_size});
    ver = 0;
  }
  // the operands follow the matrix this pass reads: the weights or their modified copy
  const uint64_t want = p.w == w_ ? w_version_ : (0x8000000000000000ull | fb_version_);
  if (ver != want) {
    eng->loadOperand(0, 0, p.w, p.wk, p.wn, s);
    ver = want;
  }
  TcEngine::Run r;
  r.in = p.in;
  r.in_ss = p.in_ss;
  r.gather = p.gather;
  r.onv = p.out_noise_vals;
  r.m = p.m;
  r.out = p.out;
  r.out_ss = p.out_ss;
  r.out_t_rows = p.out_t_rows;
  r.accumulate = p.accumulate != 0;
  r.backward = p.backward != 0;
  r.io = p.io;
  r.alpha = p.alpha;
  r.key = p.key;
  r.call = p.call;
  r.noise_id0 = p.noise_id;
  r.scale = p.scale;
  r.factor = p.factor;
  r.vnorm = p.vnorm;
  r.sval = p.sval;
  r.flags = p.flags;
  eng->run(r, s);
}

void Tile::getPulseCounters(int64_t *out_2dx) {
  if (!countsPulses()) {
    AB200_FATAL("get_pulse_counters: the device was not made with count_pulses");
  }
  const size_t size = (size_t)x_size_ * d_size_;
  if (device_ < 0) {
    std::memset(out_2dx, 0, 2 * size * sizeof(int64_t)); // no update has run without a device
    return;
  }
  requireDevice("get_pulse_counters");
  std::vector<unsigned long long> t(size);
  AB200_CUDA(cudaDeviceSynchronize());
  const unsigned long long *src[2] = {pulses_up_, pulses_down_};
  for (int q = 0; q < 2; q++) {
    AB200_CUDA(cudaMemcpy(t.data(), src[q], size * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    for (int i = 0; i < d_size_; i++) {
      for (int j = 0; j < x_size_; j++) {
        out_2dx[(size_t)q * size + (size_t)i * x_size_ + j] = (int64_t)t[(size_t)j * d_size_ + i];
      }
    }
  }
}

void Tile::lastBmStats(int32_t *n_rerun, float *max_red) {
  requireDevice("last_bm_stats");
  int h[2] = {0, 0};
  AB200_CUDA(cudaDeviceSynchronize());
  AB200_CUDA(cudaMemcpy(h, bm_stats_, sizeof(h), cudaMemcpyDeviceToHost));
  *n_rerun = h[0];
  float f;
  std::memcpy(&f, &h[1], sizeof(float));
  *max_red = h[0] > 0 ? f : 1.0f;
}

// ---------------------------------------------------------------------------------------------
// update
// ---------------------------------------------------------------------------------------------
// rows of pulse words per sample (see UpdateProblem::nseg)
static int pulseSegments(const UpEff &up) {
  if (up.pulse_type != AB200_PULSE_STOCHASTIC_COMPRESSED) {
    return 1;
  }
  return std::max(1, (up.desired_bl + kPulseSegSlots - 1) / kPulseSegSlots);
}

float Tile::pulseCountLR() const {
  // TransferRPUDevice::getPulseCountLearningRate (rpu_transfer_device.cpp:366-383)
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER && cfg_.transfer.fast_lr > 0.0f) {
    return cfg_.transfer.scale_fast_lr ? cfg_.transfer.fast_lr * lr_ : cfg_.transfer.fast_lr;
  }
  return lr_;
}

void Tile::doTransfer(cudaStream_t s) {
  // TransferRPUDevice::transfer / readAndUpdate (rpu_transfer_device.cpp:410-516): read the next
  // n_reads columns of the fast tile with one-hot inputs, write each to the slow tile by a pulsed
  // update with x = one-hot, d = read-out.
  const ab200_transfer_params &t = cfg_.transfer;
  float t_lr = t.scale_transfer_lr ? t.transfer_lr * lr_ : t.transfer_lr;
  int n = std::min(t.n_reads_per_transfer, x_size_);
  for (int k = 0; k < n; k++) {
    int col = (slice_idx_ + k) % x_size_;
    if (t_lr == 0.0f) {
      continue;
    }
    uint32_t call = transfer_calls_++;
    float write_lr = t_lr;
    bool skip_write = false;
    if (t.chopped) {
      // Tiki-Taka with choppers (ChoppedTransferRPUDevice::readAndUpdate,
      // rpu_chopped_transfer_device.cpp:357-470): plain read of the (chopped) fast tile, de-chopped
      // and accumulated in units of the buffer granularity; whole units go to the slow tile
      launchTransferRead(w_fast_, col, d_size_, t_io_, key_, call, onehot_, x_size_, tread_, 1.0f, s);
      const float from_gran = dev_[0].dw_min, to_gran = dev_[1].dw_min;
      // getBufferGranularity / getTransferLRScale (:108-142)
      float bg = t.buffer_granularity > 0.0f ? t.buffer_granularity : 1.0f;
      if (t.auto_granularity > 0.0f) {
        const float period = (float)x_size_ * fabsf(t.transfer_every);
        bg *= from_gran * t.auto_granularity / period;
      } else {
        bg *= from_gran;
      }
      float lr_scale;
      if (t.correct_gradient_magnitudes) {
        bg *= to_gran / from_gran;
        lr_scale = fabsf(t_lr) / pulseCountLR() / bg;
      } else {
        lr_scale = fabsf(t_lr) / bg;
      }
      const uint64_t n_samples = (uint64_t)std::max((int)ceilf(1.0f / std::max(t.in_chop_prob, 1e-30f)), 2);
      const uint64_t current_sample = chop_passes_ % n_samples + 1;
      if (t.dynamic) {
        // DynamicTransferRPUDevice::readAndUpdate (rpu_dynamic_transfer_device.cpp:198-343): the in
        // chopper flips at the last sample of its period (and, with in_chop_random, also by
        // chance); nothing is written during the first period
        if (t.correct_accumulation) {
          lr_scale /= std::min((float)current_sample, 1.0f / from_gran);
        }
        int flip_in = current_sample == n_samples ? 1 : 0;
        if (t.in_chop_random && chop_rng_.uniform() < t.in_chop_prob) {
          flip_in = 1;
        }
        const size_t off = (size_t)col * d_size_;
        launchTransferDynamicBuffer(t_buffer_ + off, t_mean_ + off, t_past_ + off, tread_, d_size_, lr_scale,
                                    (float)t_up_.desired_bl, t.momentum, t.forget_buffer,
                                    (float)t_up_.desired_bl * t.buffer_cap,
                                    std::min(t.tail_weightening / (float)n_samples, 1.0f),
                                    chop_switched_[col], chop_in_, col, chop_out_, flip_in, s);
        chop_switched_[col] = (unsigned char)flip_in;
        skip_write = chop_passes_ <= n_samples;
      } else {
        // the in chopper of this line flips after the transfer: always / never / at random / every
        // n-th pass over the matrix (:439-452); the host decides, the kernel flips
        int flip_in = 0;
        if (t.in_chop_prob > 0.0f) {
          if (t.in_chop_random) {
            flip_in = chop_rng_.uniform() < t.in_chop_prob ? 1 : 0;
          } else {
            flip_in = current_sample == n_samples ? 1 : 0;
          }
        }
        launchTransferChopBuffer(t_buffer_ + (size_t)col * d_size_, tread_, d_size_, lr_scale,
                                 (float)t_up_.desired_bl, t.momentum, t.forget_buffer, t.no_buffer,
                                 chop_in_, col, chop_out_, flip_in, s);
      }
      write_lr = t.step * to_gran;
      if (col == x_size_ - 1) {
        // the dynamic form never flips the out choppers (rpu_dynamic_transfer_device.cpp:326-343)
        if (t.out_chop_prob > 0.0f && !t.dynamic) {
          launchFlipChoppers(chop_out_, d_size_, t.out_chop_prob, key_, call, s);
        }
        chop_passes_++;
      }
    } else if (t.buffered) {
      // Tiki-Taka v2 (BufferedTransferRPUDevice::readAndUpdate,
      // rpu_buffered_transfer_device.cpp:142-212): plain read, accumulate into the buffer column,
      // pulse the slow tile with the whole steps only, each worth `step` granularities
      launchTransferRead(w_fast_, col, d_size_, t_io_, key_, call, onehot_, x_size_, tread_, 1.0f, s);
      const float gran = dev_[1].dw_min;
      launchTransferBuffer(t_buffer_ + (size_t)col * d_size_, tread_, d_size_, fabsf(t_lr),
                           t.thres_scale * gran, (float)t_up_.desired_bl, t.momentum,
                           t.forget_buffer, s);
      write_lr = t.step * gran;
    } else {
      launchTransferRead(w_fast_, col, d_size_, t_io_, key_, call, onehot_, x_size_, tread_, -1.0f, s);
    }
    if (skip_write) {
      continue;
    }
    UpdateProblem u{};
    u.x = onehot_;
    u.x_ss = x_size_;
    u.x_fs = 1;
    u.x_real = x_size_;
    u.d = tread_;
    u.d_ss = d_size_;
    u.d_fs = 1;
    u.x_size = x_size_;
    u.d_size = d_size_;
    u.m = 1;
    u.lr = fabsf(write_lr);
    u.lr_neg = write_lr < 0.0f;
    u.dw_min = dev_[1].dw_min;
    u.up = t_up_;
    u.nseg = pulseSegments(t_up_);
    u.key = key_;
    u.call = 0x40000000u + call;
    // own scratch: the gradient batch's pulse words are still in use when a transfer falls in
    // the middle of a batch
    u.xw = t_words_;
    u.dw = t_words_ + (size_t)u.nseg * x_size_;
    u.w = w_;
    u.par4 = dev_[1].par4;
    u.par2 = dev_[1].par2;
    u.kind = dev_[1].kind;
    u.dw_min_std = dev_[1].dw_min_std;
    u.es0 = dev_[1].es0;
    u.es1 = dev_[1].es1;
    u.pw = dev_[1].pw;
    u.pw_n = dev_[1].pw_n;
    u.mult_noise = dev_[1].mult_noise;
    u.s_begin = 0;
    u.s_end = 1;
    if (t_up_.pulse_type == AB200_PULSE_NONE) {
      launchFPUpdate(u, write_lr, s);
    } else {
      launchPulsePrepare(u, s);
      launchPulsedUpdate(u, s);
    }
  }
  slice_idx_ = (slice_idx_ + n) % x_size_;
}

void Tile::update(const float *x, const float *d, bool bias, int m, bool x_trans, bool d_trans,
                  cudaStream_t s) {
  const int x_in = x_size_ - (bias ? 1 : 0);
  updateCore(x, x_trans ? 1 : x_in, x_trans ? m : 1, x_in, d, d_trans ? 1 : d_size_,
             d_trans ? m : 1, m, s);
}

// used by the mapped array: update from sub-blocks of wider activation / gradient matrices
void Tile::updateStrided(const float *x, long long x_ss, const float *d, long long d_ss, int m,
                         cudaStream_t s) {
  updateCore(x, x_ss, 1, x_size_, d, d_ss, 1, m, s);
}

void Tile::updateCore(const float *x, long long x_ss, long long x_fs, int x_in, const float *d,
                      long long d_ss, long long d_fs, int m, cudaStream_t s) {
  requireDevice("update");
  if (m <= 0 || lr_ == 0.0f) {
    return; // "if (!learning_rate) return" (rpu_weight_updater.cpp:206-208)
  }
  ensureScratch(m * pulseSegments(up_));
  if (!delta_w_) {
    w_version_++;
  }
  UpdateProblem u{};
  u.x = x;
  u.x_ss = x_ss;
  u.x_fs = x_fs;
  u.x_real = x_in;
  u.d = d;
  u.d_ss = d_ss;
  u.d_fs = d_fs;
  u.x_size = x_size_;
  u.d_size = d_size_;
  u.m = m;
  u.key = key_;
  u.call = upd_calls_++;
  u.xw = xw_;
  u.dw = dw_;
  u.s_begin = 0;
  u.s_end = m;

  if (cfg_.mixed.enabled) {
    // the compound updates directly, whatever the pulse type (rpu_weight_updater.cpp:212-216)
    if (delta_w_) {
      AB200_FATAL("set_delta_weights is not implemented for the mixed-precision compound");
    }
    updateMixed(u, s);
    return;
  }
  const bool fp_update = cfg_.device_kind == AB200_DEVICE_IDEAL || up_.pulse_type == AB200_PULSE_NONE;
  if (fp_update) {
    if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
      AB200_FATAL("Transfer with PulseType::None is not implemented");
    }
    if (delta_w_) {
      // delta-weight mode: the gradient itself, +sum d x (bwd_alpha = 1), replaces the buffer
      u.w = delta_w_;
      launchFPUpdate(u, -1.0f, s, /*overwrite=*/true);
      return;
    }
    u.w = w_;
    launchFPUpdate(u, lr_, s);
    return;
  }
  if (delta_w_) {
    AB200_FATAL("set_delta_weights is implemented for the floating-point update only");
  }
  if (up_.pulse_type == AB200_PULSE_NONE_WITH_DEVICE) {
    if (cfg_.device_kind == AB200_DEVICE_TRANSFER) {
      AB200_FATAL("Transfer with PulseType::NoneWithDevice is not implemented");
    }
    u.w = w_;
    u.par4 = dev_[0].par4;
    launchFPUpdate(u, lr_, s, /*overwrite=*/false, /*clip_each=*/true);
    return;
  }

  const float pc_lr = pulseCountLR();
  u.lr = fabsf(pc_lr);
  u.lr_neg = pc_lr < 0.0f;
  u.up = up_;
  u.nseg = pulseSegments(up_);
  u.dw_min = dev_[0].dw_min;
  u.par4 = dev_[0].par4;
  u.par2 = dev_[0].par2;
  u.kind = dev_[0].kind;
  u.dw_min_std = dev_[0].dw_min_std;
  u.es0 = dev_[0].es0;
  u.es1 = dev_[0].es1;
  u.pw = dev_[0].pw;
  u.pw_n = dev_[0].pw_n;
  u.mult_noise = dev_[0].mult_noise;
  if (cfg_.device_kind == AB200_DEVICE_TRANSFER && cfg_.transfer.chopped) {
    u.chop_x = chop_in_;
    u.chop_d = chop_out_;
  }
  u.gather = upd_gather_;
  launchPulsePrepare(u, s);
  const bool stream_upd = streamUpdateEligible(u);
  const int m_pad = (m * u.nseg + 31) / 32 * 32;
  if (stream_upd) {
    ensureStreamScratch(m_pad);
    launchPulseTranspose(u, xwt_, xnzt_, m_pad, s);
    launchPulseCompact(u, xwt_, xnzt_, m_pad, xls_, xlx_, xloff_, s);
  }
  auto applyRange = [&](UpdateProblem &r) {
    if (stream_upd) {
      launchPulsedUpdateStream(r, xwt_, xnzt_, m_pad, s, xls_, xlx_, xloff_);
    } else {
      launchPulsedUpdate(r, s);
    }
  };

  if (cfg_.device_kind != AB200_DEVICE_TRANSFER) {
    u.w = w_;
    if (pulses_up_) {
      launchPulseCounter(u, pulses_up_, pulses_down_, s);
    }
    applyRange(u);
    return;
  }

  // Tiki-Taka: gradient pulses go to the fast tile; the batch is cut where the vector-update
  // counter reaches a multiple of the transfer period (TransferRPUDevice::finishUpdateCycle,
  // rpu_transfer_device.cpp:539-557; getTransferEvery :400-408).
  u.w = w_fast_;
  const ab200_transfer_params &t = cfg_.transfer;
  long long every = t.units_in_mbatch ? (long long)std::ceil(t.transfer_every * (float)m)
                                      : (long long)std::lround(t.transfer_every);
  if (every < 0) {
    every = 0;
  }
  int s0 = 0;
  while (s0 < m) {
    int s1 = m;
    if (every > 0) {
      long long to_next = every - (update_idx_ % every);
      if (to_next < (long long)(m - s0)) {
        s1 = s0 + (int)to_next;
      }
    }
    u.s_begin = s0;
    u.s_end = s1;
    applyRange(u);
    update_idx_ += s1 - s0;
    if (every > 0 && update_idx_ % every == 0) {
      doTransfer(s);
    }
    s0 = s1;
  }
}

// Mixed-precision compound (MixedPrecRPUDevice::doDirectVectorUpdate, rpu_mixedprec_device.cpp:
// 196-345; MixedPrecRPUDeviceBase::doTransfer / transfer, rpu_mixedprec_device_base.cpp:282-352):
// chi += lr q(d) q(x)^T sample by sample; after sample k > 0 with k % (transfer_every * m) == 0
// the next rows of chi hand their whole granularities to the device.
void Tile::updateMixed(UpdateProblem &u, cudaStream_t s) {
  const ab200_mixedprec_params &mp = cfg_.mixed;
  const int m = u.m;
  const bool quantised = mp.n_x_bins > 0 && mp.n_d_bins > 0;
  UpdateProblem a = u; // accumulation into chi
  a.w = chi_;
  a.par4 = nullptr;
  if (quantised) {
    if (m > mp_q_cap_) {
      AB200_CUDA(cudaStreamSynchronize(s));
      cudaFree(mp_qx_);
      cudaFree(mp_qd_);
      mp_qx_ = mp_qd_ = nullptr;
      const int cap = m + m / 4 + 16;
      AB200_CUDA(cudaMalloc(&mp_qx_, (size_t)cap * x_size_ * sizeof(float)));
      AB200_CUDA(cudaMalloc(&mp_qd_, (size_t)cap * d_size_ * sizeof(float)));
      mp_q_cap_ = cap;
    }
    launchMixedQuantize(u, mp.n_x_bins, mp.n_d_bins, mp.stoc_round_x, mp.stoc_round_d, mp_qx_, mp_qd_, s);
    a.x = mp_qx_;
    a.x_ss = x_size_;
    a.x_fs = 1;
    a.x_real = x_size_;
    a.d = mp_qd_;
    a.d_ss = d_size_;
    a.d_fs = 1;
  }
  const long long every = (long long)mp.transfer_every * m;
  int s0 = 0;
  while (s0 < m) {
    // the segment ends with the sample after which a transfer falls
    int s1 = m;
    if (every > 0) {
      long long k = mp_update_idx_; // index of sample s0
      long long next = k > 0 && k % every == 0 ? k : (k / every + 1) * every;
      if (next - k < (long long)(m - s0)) {
        s1 = s0 + (int)(next - k) + 1;
      }
    }
    UpdateProblem seg = a;
    seg.x = a.x + (long long)s0 * a.x_ss;
    seg.d = a.d + (long long)s0 * a.d_ss;
    seg.m = s1 - s0;
    // chi += (lr * d) * x in the order of the samples (the quantised form is a plain loop in
    // the reference; the unquantised one a BLAS rank-one update)
    launchFPUpdate(seg, -lr_, s, /*overwrite=*/false, /*clip_each=*/quantised);
    const long long last = mp_update_idx_ + (s1 - s0) - 1; // index of the segment's last sample
    mp_update_idx_ += s1 - s0;
    if (every > 0 && last > 0 && last % every == 0) {
      transferMixed(s);
    }
    s0 = s1;
  }
}

void Tile::transferMixed(cudaStream_t s) {
  const ab200_mixedprec_params &mp = cfg_.mixed;
  if (mp.n_rows_per_transfer == 0 || mp.transfer_lr == 0.0f) {
    return;
  }
  int n = mp.n_rows_per_transfer < 0 ? d_size_ : std::min(mp.n_rows_per_transfer, d_size_);
  int row0 = mp_row_idx_;
  if (mp.random_row && n < d_size_) {
    row0 = std::max(std::min((int)floorf(chop_rng_.uniform() * (float)d_size_), d_size_ - 1), 0);
  }
  if (!mp_counts_) {
    AB200_CUDA(cudaMalloc(&mp_counts_, (size_t)d_size_ * x_size_ * sizeof(float)));
    AB200_CUDA(cudaMalloc(&mp_onehot_, (size_t)d_size_ * d_size_ * sizeof(float)));
  }
  launchMixedTruncate(chi_, x_size_, d_size_, row0, n, mp_granularity_, mp_counts_, mp_onehot_, s);
  // one pulsed update with the rows as samples: every row writes only its own weights, so the
  // result is that of the reference's row-by-row updates
  UpEff up = up_;
  up.update_management = 1; // "should be both true to get the desired step" (setUpPar, :293-303)
  up.update_bl_management = 1;
  const int nseg = pulseSegments(up);
  ensureScratch(n * nseg);
  w_version_++;
  const float t_lr = mp_granularity_ * mp.transfer_lr;
  UpdateProblem u{};
  u.x = mp_counts_;
  u.x_ss = x_size_;
  u.x_fs = 1;
  u.x_real = x_size_;
  u.d = mp_onehot_;
  u.d_ss = d_size_;
  u.d_fs = 1;
  u.x_size = x_size_;
  u.d_size = d_size_;
  u.m = n;
  u.key = key_;
  u.call = 0x40000000u + transfer_calls_++;
  u.xw = xw_;
  u.dw = dw_;
  u.w = w_;
  u.s_begin = 0;
  u.s_end = n;
  u.par4 = dev_[0].par4;
  if (up.pulse_type == AB200_PULSE_NONE) {
    launchFPUpdate(u, t_lr, s);
  } else if (up.pulse_type == AB200_PULSE_NONE_WITH_DEVICE) {
    launchFPUpdate(u, t_lr, s, /*overwrite=*/false, /*clip_each=*/true);
  } else {
    u.lr = fabsf(t_lr);
    u.lr_neg = t_lr < 0.0f;
    u.up = up;
    u.nseg = nseg;
    u.dw_min = dev_[0].dw_min;
    u.par2 = dev_[0].par2;
    u.kind = dev_[0].kind;
    u.dw_min_std = dev_[0].dw_min_std;
    u.es0 = dev_[0].es0;
    u.es1 = dev_[0].es1;
    u.pw = dev_[0].pw;
    u.pw_n = dev_[0].pw_n;
    u.mult_noise = dev_[0].mult_noise;
    launchPulsePrepare(u, s);
    launchPulsedUpdate(u, s);
  }
  mp_row_idx_ = (row0 + n) % d_size_;
}

void Tile::coincidences(const float *x, const float *d, int32_t *counts, cudaStream_t s) {
  requireDevice("coincidences");
  if (cfg_.device_kind == AB200_DEVICE_IDEAL || up_.pulse_type == AB200_PULSE_NONE ||
      up_.pulse_type == AB200_PULSE_NONE_WITH_DEVICE) {
    AB200_FATAL("coincidences need a pulsed update");
  }
  ensureScratch(pulseSegments(up_));
  UpdateProblem u{};
  u.x = x;
  u.x_ss = x_size_;
  u.x_fs = 1;
  u.x_real = x_size_;
  u.d = d;
  u.d_ss = d_size_;
  u.d_fs = 1;
  u.x_size = x_size_;
  u.d_size = d_size_;
  u.m = 1;
  const float pc_lr = pulseCountLR();
  u.lr = fabsf(pc_lr);
  u.lr_neg = pc_lr < 0.0f;
  u.up = up_;
  u.nseg = pulseSegments(up_);
  u.dw_min = dev_[0].dw_min;
  u.key = key_;
  u.call = 0x7fffffffu;
  u.xw = xw_;
  u.dw = dw_;
  launchPulsePrepare(u, s);
  launchCoincidences(u, counts, s);
}

// ---------------------------------------------------------------------------------------------
// host-buffer entry points: pinned staging + H2D, kernels, D2H, all on the caller's stream
// ---------------------------------------------------------------------------------------------
void Tile::forwardHost(const float *x, float *d, bool bias, int m, bool x_trans, bool d_trans,
                       bool is_test, cudaStream_t s) {
  requireDevice("forward");
  const size_t nx = (size_t)m * (x_size_ - (bias ? 1 : 0)), nd = (size_t)m * d_size_;
  ensureStage(nx + nd);
  std::memcpy(stage_pinned_, x, nx * sizeof(float));
  AB200_CUDA(cudaMemcpyAsync(stage_dev_, stage_pinned_, nx * sizeof(float), cudaMemcpyHostToDevice, s));
  forward(stage_dev_, stage_dev_ + nx, bias, m, x_trans, d_trans, is_test, s);
  AB200_CUDA(cudaMemcpyAsync(stage_pinned_ + nx, stage_dev_ + nx, nd * sizeof(float),
                             cudaMemcpyDeviceToHost, s));
  AB200_CUDA(cudaStreamSynchronize(s));
  std::memcpy(d, stage_pinned_ + nx, nd * sizeof(float));
}

void Tile::backwardHost(const float *d, float *x, bool bias, int m, bool d_trans, bool x_trans,
                        cudaStream_t s) {
  requireDevice("backward");
  const size_t nx = (size_t)m * (x_size_ - (bias ? 1 : 0)), nd = (size_t)m * d_size_;
  ensureStage(nx + nd);
  std::memcpy(stage_pinned_, d, nd * sizeof(float));
  AB200_CUDA(cudaMemcpyAsync(stage_dev_, stage_pinned_, nd * sizeof(float), cudaMemcpyHostToDevice, s));
  backward(stage_dev_, stage_dev_ + nd, bias, m, d_trans, x_trans, s);
  AB200_CUDA(cudaMemcpyAsync(stage_pinned_ + nd, stage_dev_ + nd, nx * sizeof(float),
                             cudaMemcpyDeviceToHost, s));
  AB200_CUDA(cudaStreamSynchronize(s));
  std::memcpy(x, stage_pinned_ + nd, nx * sizeof(float));
}

void Tile::updateHost(const float *x, const float *d, bool bias, int m, bool x_trans, bool d_trans,
                      cudaStream_t s) {
  requireDevice("update");
  const size_t nx = (size_t)m * (x_size_ - (bias ? 1 : 0)), nd = (size_t)m * d_size_;
  ensureStage(nx + nd);
  std::memcpy(stage_pinned_, x, nx * sizeof(float));
  std::memcpy(stage_pinned_ + nx, d, nd * sizeof(float));
  AB200_CUDA(cudaMemcpyAsync(stage_dev_, stage_pinned_, (nx + nd) * sizeof(float),
                             cudaMemcpyHostToDevice, s));
  update(stage_dev_, stage_dev_ + nx, bias, m, x_trans, d_trans, s);
  AB200_CUDA(cudaStreamSynchronize(s));
}

} // namespace ab200
