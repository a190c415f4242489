/*
 * aihwkit_b200 — C ABI of the B200-native analog-tile hot path.
 *
 * Every entry point is plain C: opaque handles, raw pointers, sizes and a
 * CUDA stream passed as `void *` (a `cudaStream_t`; NULL = legacy default
 * stream). No torch / pybind types cross this boundary.  The functions are the
 * ones the reference's Python binding (`aihwkit.simulator.rpu_base`) would
 * bind for the analog tile; each declaration cites the reference interface it
 * replaces as `file:line` relative to the aihwkit source tree.
 *
 * Conventions
 *  - x_size = tile inputs (columns), d_size = tile outputs (rows), m_batch =
 *    number of input vectors per call.
 *  - Host weight matrices at this API are row-major [d_size][x_size]
 *    (src/rpucuda/rpu.cpp:227-236). On the device the tile keeps fp32 master
 *    weights as [x_size][d_size] like the reference GPU tile
 *    (src/rpucuda/cuda/rpucuda.cu:285-299).
 *  - Activations: "batch first iff *_trans" (src/rpucuda/rpu.h:415-417):
 *    x_trans == 0 -> X is [m_batch][x_size]; x_trans != 0 -> X is
 *    [x_size][m_batch]; likewise for D.
 *  - All entry points return 0 on success. On failure they return a non-zero
 *    code and ab200_last_error() gives the message the reference would have
 *    thrown as std::runtime_error (src/rpucuda/utility_functions.h:63-69).
 *  - There is no CPU compute path: every compute call needs a CUDA device.
 */
#ifndef AIHWKIT_B200_H_
#define AIHWKIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums: numeric values follow src/rpucuda/rpu_pulsed_meta_parameter.h:146-178 ---- */
enum ab200_noise_management {
  AB200_NM_NONE = 0,
  AB200_NM_ABS_MAX = 1,
  AB200_NM_ABS_MAX_NP_SUM = 2,
  AB200_NM_MAX = 3,
  AB200_NM_CONSTANT = 4,
  AB200_NM_AVERAGE_ABS_MAX = 5,
  AB200_NM_AVERAGE_ABS_MAX_SINGLE_VALUE = 6,
  AB200_NM_ABS_MAX_SINGLE_VALUE = 7
};
enum ab200_bound_management {
  AB200_BM_NONE = 0,
  AB200_BM_ITERATIVE = 1,
  AB200_BM_ITERATIVE_WORST_CASE = 2
};
enum ab200_w_noise_type {
  AB200_WNOISE_NONE = 0,
  AB200_WNOISE_ADDITIVE_CONSTANT = 1,
  AB200_WNOISE_PCM_READ = 2
};
enum ab200_pulse_type {
  AB200_PULSE_NONE = 0,
  AB200_PULSE_STOCHASTIC_COMPRESSED = 1,
  AB200_PULSE_STOCHASTIC = 2,
  AB200_PULSE_NONE_WITH_DEVICE = 3,
  AB200_PULSE_MEAN_COUNT = 4,
  AB200_PULSE_DETERMINISTIC_IMPLICIT = 5
};
enum ab200_device_kind {
  AB200_DEVICE_IDEAL = 0,                 /* SimpleRPUDevice: floating-point update */
  AB200_DEVICE_CONSTANT_STEP = 1,         /* rpu_constantstep_device.h */
  AB200_DEVICE_LINEAR_STEP = 2,           /* rpu_linearstep_device.h */
  AB200_DEVICE_SOFT_BOUNDS = 3,           /* rpu_linearstep_device.h:70-83 */
  AB200_DEVICE_SOFT_BOUNDS_REFERENCE = 4, /* rpu_softbounds_reference_device.h */
  AB200_DEVICE_TRANSFER = 5,              /* rpu_transfer_device.h (Tiki-Taka) */
  AB200_DEVICE_EXP_STEP = 6,              /* rpu_expstep_device.h */
  AB200_DEVICE_POW_STEP = 7,              /* rpu_powstep_device.h */
  AB200_DEVICE_PIECEWISE_STEP = 8         /* rpu_piecewisestep_device.h */
};

/* largest number of nodes of the PiecewiseStep interpolation tables */
#define AB200_PIECEWISE_MAX_NODES 32

/* IOMetaParameter (src/rpucuda/rpu_pulsed_meta_parameter.h:180-226); attribute names as
 * bound in src/aihwkit/simulator/rpu_base_src/rpu_base_devices.cpp:485-519.
 * inp_res / out_res are the user-facing values (e.g. 1/126); the library applies
 * res <- checkRes(res) * 2 * bound exactly once, like initializeForForward
 * (src/rpucuda/rpu_pulsed_meta_parameter.cpp:26-37,56-57). */
typedef struct ab200_io_params {
  int32_t is_perfect;
  int32_t noise_management; /* enum ab200_noise_management */
  int32_t bound_management; /* enum ab200_bound_management */
  int32_t w_noise_type;     /* enum ab200_w_noise_type */
  int32_t bm_test_negative_bound;
  int32_t max_bm_factor;
  int32_t inp_sto_round;
  int32_t out_sto_round;
  float inp_bound;
  float inp_res;
  float inp_noise;
  float out_bound;
  float out_res;
  float out_noise;
  float out_scale;
  float w_noise;
  float nm_thres;
  float max_bm_res;
  float inp_asymmetry;
  float out_asymmetry;
  float nm_assumed_wmax; /* AbsMaxNPSum noise management / IterativeWorstCase bound management */
  /* relative spread of the output noise over the output lines: line i keeps
   * |out_noise * (1 + out_noise_std * N(0,1))| for the life of the tile
   * (rpu_forward_backward_pass.cpp:306-313, :696) */
  float out_noise_std;
  /* AverageAbsMax noise management: weight of a sample's abs-max in the running value
   * s <- s (1 - nm_decay) + nm_decay * max|x| (rpu_forward_backward_pass.cpp:139-150) */
  float nm_decay;
  /* Non-idealities of the analog output lines, CUDA-core kernels only
   * (rpu_forward_backward_pass.cpp:388-517, :673-719; bound as ir_drop, ir_drop_g_ratio,
   * v_offset_std, r_series, out_nonlinearity, out_nonlinearity_std, slope_calibration):
   *  - IR drop: y_i -= ir_drop * c_i * sum_j w_ij v_j (1 - (1 - j/n)^2), c_i a cubic of the line
   *    current a_i = n / ir_drop_g_ratio * sum_j |w_ij| |v_j|;
   *  - voltage offsets and series resistance: y_i = (1 - vo_i) y_i / (1 + min(r_series |y_i|,
   *    r_series_max_total)), vo_i = max(v_offset_std N(0,1), 0) per line;
   *  - output non-linearity: y_i = f y_i / (1 + |nl_i y_i|), nl_i = |out_nonlinearity / out_bound *
   *    (1 + out_nonlinearity_std N(0,1))| per line, f the slope calibration factor.
   * The per-line values are drawn once per tile and direction; ab200_tile_get_io_vector /
   * ab200_tile_set_io_vector read and replace them. r_series_max_total <= 0 means no limit. */
  float ir_drop;
  float ir_drop_g_ratio;
  float v_offset_std;
  float r_series;
  float r_series_max_total;
  float out_nonlinearity;
  float out_nonlinearity_std;
  float slope_calibration;
  /* AnalogMVType (src/rpucuda/rpu_pulsed_meta_parameter.h:41-48, computeAnalogMV
   * rpu_forward_backward_pass.cpp:820-876): ONE_PASS, or the negative and the positive inputs in
   * two passes through the array, each with its own analog non-idealities and weight noise; the
   * two results are added before the output stage (POS_NEG_SEPARATE: one output noise draw, one
   * ADC conversion of the sum) or after it (POS_NEG_SEPARATE_DIGITAL_SUM: each pass converted on
   * its own, bound management needs both inside the bound). CUDA-core kernels only. */
  int32_t mv_type; /* enum ab200_mv_type */
} ab200_io_params;

/* AnalogMVType::Ideal of the reference is is_perfect = 1 here */
enum ab200_mv_type {
  AB200_MV_ONE_PASS = 0,
  AB200_MV_POS_NEG_SEPARATE = 1,
  AB200_MV_POS_NEG_SEPARATE_DIGITAL_SUM = 2
};

/* PulsedUpdateMetaParameter (src/rpucuda/rpu_pulsed_meta_parameter.h:248-279;
 * rpu_base_devices.cpp:469-483). */
typedef struct ab200_update_params {
  int32_t pulse_type; /* enum ab200_pulse_type */
  int32_t desired_bl;
  int32_t fixed_bl;
  int32_t update_management;
  int32_t update_bl_management;
  int32_t sto_round;
  float um_grad_scale;
  float res;
  float x_res_implicit;
  float d_res_implicit;
} ab200_update_params;

/* DriftParameter (src/rpucuda/weight_drifter.h:17-60; bound in rpu_base_devices.cpp:521-533 as nu,
 * nu_dtod, nu_std, wg_ratio, g_offset, w_offset, nu_k, log_g0, t_0, reset_tol, w_noise_std):
 * power-law drift w(t) = w0 * (t / t0)^(-nu) of weights that were not written since. A zeroed
 * struct means "no drift" (t0, wg_ratio and reset_tol of 0 read as 1, 1 and 1e-7). */
typedef struct ab200_drift_params {
  float nu;
  float nu_dtod;
  float nu_std;
  float wg_ratio;
  float g_offset;
  float w_offset;
  float nu_k;
  float log_g0;
  float t0;
  float reset_tol;
  float w_read_std;
} ab200_drift_params;

/* One pulsed device (PulsedRPUDeviceMetaParameter, src/rpucuda/rpu_pulsed_device.h:60-110,
 * plus the LinearStep / SoftBoundsReference extras: rpu_linearstep_device.h:24-58,
 * rpu_softbounds_reference_device.h:17-42). */
typedef struct ab200_device_params {
  int32_t kind; /* enum ab200_device_kind, one of the single-device kinds */
  uint32_t construction_seed;
  int32_t enforce_consistency;
  int32_t dw_min_dtod_log_normal;
  int32_t perfect_bias;
  /* count the pulses every weight receives, up and down apart (count_pulses,
   * src/rpucuda/rpu_pulsed_device.h:91; the reference counts on its GPU tile only,
   * cuda/rpucuda_pulsed_device.cu:470-492, cuda/pwu_kernel.h:1523-1620): read with
   * ab200_tile_get_pulse_counters. Single devices and the pulsed update only. */
  int32_t count_pulses;
  float dw_min;
  float dw_min_dtod;
  float dw_min_std;
  float w_min;
  float w_min_dtod;
  float w_max;
  float w_max_dtod;
  float up_down;
  float up_down_dtod;
  /* LinearStep / SoftBounds */
  int32_t ls_mult_noise;
  int32_t ls_allow_increasing_slope;
  int32_t ls_mean_bound_reference;
  float ls_decrease_up;
  float ls_decrease_down;
  float ls_decrease_up_dtod;
  float ls_decrease_down_dtod;
  /* SoftBoundsReference */
  int32_t mult_noise;
  int32_t subtract_symmetry_point;
  float slope_up_dtod;
  float slope_down_dtod;
  float reference_mean;
  float reference_std;
  /* decay / diffusion / reset (SimpleMetaParameter lifetime, diffusion; PulsedRPUDeviceMetaParameter
   * lifetime_dtod, diffusion_dtod, reset, reset_dtod; reset_std; rpu_pulsed_device.h:70-85,
   * rpu_simple_device.h:40-90) */
  float lifetime;
  float lifetime_dtod;
  float diffusion;
  float diffusion_dtod;
  float reset;
  float reset_dtod;
  float reset_std;
  /* ExpStep (ExpStepRPUDeviceMetaParameter, rpu_expstep_device.h:22-29; bound as A_up, A_down,
   * gamma_up, gamma_down, a, b, dw_min_std_add, dw_min_std_slope) */
  float es_A_up;
  float es_A_down;
  float es_gamma_up;
  float es_gamma_down;
  float es_a;
  float es_b;
  float dw_min_std_add;
  float dw_min_std_slope;
  /* PowStep (PowStepRPUDeviceMetaParameter, rpu_powstep_device.h:22-25; bound as pow_gamma,
   * pow_gamma_dtod, pow_up_down, pow_up_down_dtod) */
  float ps_gamma;
  float ps_gamma_dtod;
  float ps_gamma_up_down;
  float ps_gamma_up_down_dtod;
  /* PiecewiseStep (PiecewiseStepRPUDeviceMetaParameter, rpu_piecewisestep_device.h:17-50; bound as
   * piecewise_up, piecewise_down): the step is dw_min times a factor interpolated linearly
   * between pw_n equally spaced nodes over [w_min, w_max] of the element */
  int32_t pw_n;
  float pw_up[AB200_PIECEWISE_MAX_NODES];
  float pw_down[AB200_PIECEWISE_MAX_NODES];
  /* drift of the device (SimpleRPUDeviceMetaParameter::drift, rpu_simple_device.h); for
   * AB200_DEVICE_IDEAL the tile's own simple drift (RPUSimple::driftWeights, rpu.cpp:1581-1587) */
  ab200_drift_params drift;
} ab200_device_params;

/* TransferRPUDeviceMetaParameter (src/rpucuda/rpu_transfer_device.h:52-75). */
typedef struct ab200_transfer_params {
  float gamma;
  float transfer_every;
  int32_t units_in_mbatch;
  int32_t n_reads_per_transfer;
  float fast_lr;
  float transfer_lr;
  int32_t scale_transfer_lr;
  int32_t scale_fast_lr;
  int32_t transfer_columns;
  ab200_io_params transfer_io;
  ab200_update_params transfer_up;
  /* BufferedTransferRPUDeviceMetaParameter (Tiki-Taka v2, src/rpucuda/rpu_buffered_transfer_device.h:
   * 20-37): the read-out of the fast tile is accumulated in a digital buffer per element, and
   * the slow tile is pulsed only by the whole multiples of thres_scale * granularity in it */
  int32_t buffered;
  int32_t forget_buffer;
  float thres_scale;
  float step;
  float momentum;
  /* ChoppedTransferRPUDeviceMetaParameter (Tiki-Taka with choppers,
   * src/rpucuda/rpu_chopped_transfer_device.h:22-40; needs buffered = 1, one read per transfer): the
   * gradient pulses of input line j and output line i reach the fast tile with the sign
   * in_chopper[j] xor out_chopper[i]; a transfer de-chops its read with the same signs and
   * accumulates it in units of the buffer granularity (whole units are written to the slow
   * tile); the in chopper of the transferred line then flips with probability in_chop_prob (at
   * random, or every ceil(1 / in_chop_prob) passes over the matrix when in_chop_random = 0), the
   * out choppers with probability out_chop_prob after every full pass. auto_scale and a negative
   * transfer_every (automatic period) are not implemented. */
  int32_t chopped;
  int32_t in_chop_random;
  int32_t correct_gradient_magnitudes;
  int32_t no_buffer;
  float in_chop_prob;
  float out_chop_prob;
  float auto_granularity;
  float buffer_granularity;
  /* DynamicTransferRPUDeviceMetaParameter (Tiki-Taka with choppers and a dynamically estimated
   * reference, src/rpucuda/rpu_dynamic_transfer_device.h:26-36; needs chopped = 1 and
   * in_chop_prob > 0): every element keeps a running mean of its reads (weight of a new read
   * min(tail_weightening / n_samples, 1), n_samples = max(ceil(1 / in_chop_prob), 2)); when the
   * in chopper of a line has flipped, the mean becomes the reference that later reads of the
   * line are taken against. Writes start after n_samples passes over the matrix. With
   * forget_buffer = 0 the buffer is clamped to buffer_cap * desired_bl of the transfer update
   * (buffer_cap <= 0: no clamp). correct_accumulation divides the transfer scale by
   * min(sample index within the chopper period, 1 / fast granularity). The reference's
   * experimental_fast_lr_feedback (not reachable through its Python bindings) is not built. */
  int32_t dynamic;
  int32_t correct_accumulation;
  float tail_weightening;
  float buffer_cap;
} ab200_transfer_params;

/* MixedPrecRPUDeviceMetaParameter (src/rpucuda/rpu_mixedprec_device.h:30-37,
 * rpu_mixedprec_device_base.h:24-35; Nandakumar et al. 2020): the rank-one update of every sample
 * is computed digitally, chi += lr * q(d) q(x)^T with x and d quantised to n_x_bins / n_d_bins
 * levels of their abs-max (rint, optionally stochastic), and kept in a matrix chi. After sample
 * k > 0 with k % (transfer_every * m_batch) == 0, n_rows_per_transfer rows (< 0: all) starting
 * at a running row index (random_row: drawn) move their whole multiples of the granularity
 * (0: that of the device) to the analog device `device[0]` by a pulsed update with update
 * management and update BL management on and learning rate granularity * transfer_lr.
 * device_kind names the analog device. Quantising only one of x and d is not built (both
 * counts positive, or both <= 0 for the unquantised outer product). set_weights clears chi and
 * the counters. chi is the last hidden parameter, "hidden_weights_chi". */
typedef struct ab200_mixedprec_params {
  int32_t enabled;
  int32_t transfer_every;
  int32_t n_rows_per_transfer;
  int32_t random_row;
  float granularity;
  int32_t n_x_bins;
  int32_t n_d_bins;
  int32_t stoc_round_x;
  int32_t stoc_round_d;
  float transfer_lr;
} ab200_mixedprec_params;

/* Everything PulsedMetaParameter::createRPUArray needs
 * (src/rpucuda/rpu_pulsed.cpp:49-56; rpu_base_devices.cpp:453-467). */
typedef struct ab200_tile_config {
  int32_t x_size;
  int32_t d_size;
  ab200_io_params forward_io;
  ab200_io_params backward_io;
  ab200_update_params update;
  int32_t device_kind;          /* enum ab200_device_kind */
  ab200_device_params device[2]; /* [0] only, or fast/slow pair for TRANSFER */
  ab200_transfer_params transfer;
  ab200_mixedprec_params mixed; /* enabled = 0 unless the device is a mixed-precision compound */
  uint64_t seed;                /* Philox key for all run-time noise of this tile */
} ab200_tile_config;

typedef struct ab200_tile ab200_tile;
typedef struct ab200_array ab200_array;

/* Message of the last failed call on this thread (never NULL). */
const char *ab200_last_error(void);
/* Library version string. */
const char *ab200_version(void);
/* sizeof of the parameter structs as the library was compiled (0 io, 1 update, 2 device,
 * 3 transfer, 4 tile config, 5 scatter plan, 6 mixed precision): lets a foreign-language binding
 * check its own layout. */
size_t ab200_sizeof(int which);

/* Fill the structs with the reference's defaults (IOMetaParameter / PulsedUpdateMetaParameter /
 * PulsedRPUDeviceMetaParameter default member initialisers). */
void ab200_default_io_params(ab200_io_params *io);
void ab200_default_update_params(ab200_update_params *up);
void ab200_default_device_params(ab200_device_params *dp, int32_t kind);
void ab200_default_transfer_params(ab200_transfer_params *tp);
void ab200_default_mixedprec_params(ab200_mixedprec_params *mp); /* enabled = 0 */

/* ---- tile life cycle ------------------------------------------------------------------- */

/* Replaces PulsedMetaParameter::createRPUArray + RPUCudaPulsed construction
 * (src/rpucuda/rpu_pulsed.cpp:49-56, src/rpucuda/cuda/rpucuda_pulsed.cu:69-88): draws the
 * per-element device parameters on the host, uploads them to `cuda_device`, weights start at 0. */
int ab200_tile_create(const ab200_tile_config *cfg, int cuda_device, ab200_tile **out);
int ab200_tile_destroy(ab200_tile *tile);
/* CudaAnalogTile(cpu_tile) (src/aihwkit/simulator/rpu_base_src/rpu_base_tiles_cuda.cpp:532-538):
 * a tile created with cuda_device = -1 only carries configuration, weights and the host-drawn
 * device parameters; this uploads it. Compute calls on a tile without a device fail. */
int ab200_tile_to_device(ab200_tile *tile, int cuda_device);

int ab200_tile_get_x_size(const ab200_tile *tile); /* rpu.h getXSize */
int ab200_tile_get_d_size(const ab200_tile *tile); /* rpu.h getDSize */

/* RPUSimple::setLearningRate / getLearningRate (src/rpucuda/rpu.h:246-249). */
int ab200_tile_set_learning_rate(ab200_tile *tile, float lr);
int ab200_tile_get_learning_rate(const ab200_tile *tile, float *lr);

/* RPUPulsed::setWeights (src/rpucuda/rpu_pulsed.cpp:288-292): host [d][x]; clipped to the
 * per-element bounds of the device.  RPUSimple::getWeights (src/rpucuda/rpu.cpp:1308-1314). */
int ab200_tile_set_weights(ab200_tile *tile, const float *w_host);
int ab200_tile_get_weights(ab200_tile *tile, float *w_host);
/* Device-resident [x_size][d_size] variants (get_weights_cuda / set_weights_cuda probed by
 * src/aihwkit/simulator/tiles/base.py:452-453). */
int ab200_tile_set_weights_device(ab200_tile *tile, const float *w_dev_xd, void *stream);
int ab200_tile_get_weights_device(ab200_tile *tile, float *w_dev_xd, void *stream);
/* RPUCudaSimple::setSharedWeights (src/rpucuda/cuda/rpucuda.cu:322-334): alias caller-owned
 * fp32 [x_size][d_size] device memory as the master weights. `version` is any counter that
 * changes when the caller modified the buffer (operand caches are rebuilt when (ptr, version)
 * changes). */
int ab200_tile_set_shared_weights(ab200_tile *tile, float *w_dev_xd, uint64_t version);
/* RPUSimple::setDeltaWeights / reset_delta_weights (src/rpucuda/rpu.cpp:1459-1481, bound at
 * src/aihwkit/simulator/rpu_base_src/rpu_base_tiles.cpp:231-257): while a caller-owned fp32
 * [x_size][d_size] device buffer is set, the floating-point update leaves the weights alone and
 * overwrites the buffer with the gradient sum_s d_s x_s / bwd_alpha (getAlphaLearningRate
 * rpu.cpp:1400-1403, getUpBeta :1509-1511) - the update path of hardware-aware training
 * (tiles/functions.py:91-102). Null ends the mode. */
int ab200_tile_set_delta_weights(ab200_tile *tile, float *dw_dev_xd);

/* Hidden (per-element device) parameters: RPUPulsed::getDeviceParameterNames / getDeviceParameter /
 * setDeviceParameter (src/rpucuda/rpu_pulsed.cpp:330-380; rpu_base_tiles.cpp:764-825).
 * Arrays are host [n][d][x]. */
int ab200_tile_hidden_parameter_count(const ab200_tile *tile);
const char *ab200_tile_hidden_parameter_name(const ab200_tile *tile, int index);
int ab200_tile_get_hidden_parameters(ab200_tile *tile, float *out_host);
int ab200_tile_set_hidden_parameters(ab200_tile *tile, const float *in_host);

/* ---- the hot path ---------------------------------------------------------------------- */

/* RPUSimple::forward (src/rpucuda/rpu.h:418-425; rpu.cpp:509-533) with the IO-managed MVM of
 * ForwardBackwardPassIOManaged::forwardVector (rpu_forward_backward_pass.cpp:901-988).
 * x_dev, d_dev: device pointers. bias != 0 appends a constant-1 input (rpu.cpp:636-648). */
int ab200_tile_forward(ab200_tile *tile, const float *x_dev, float *d_dev, int bias, int m_batch,
                       int x_trans, int d_trans, int is_test, void *stream);
/* RPUSimple::backward (rpu.h:426-432; rpu_forward_backward_pass.cpp:991-1027). */
int ab200_tile_backward(ab200_tile *tile, const float *d_dev, float *x_dev, int bias, int m_batch,
                        int d_trans, int x_trans, void *stream);
/* RPUSimple::update (rpu.h:433-439) -> PulsedRPUWeightUpdater::updateVectorWithDevice
 * (rpu_weight_updater.cpp:198-294) for every sample of the batch, in batch order. */
int ab200_tile_update(ab200_tile *tile, const float *x_dev, const float *d_dev, int bias,
                      int m_batch, int x_trans, int d_trans, void *stream);

/* Same three calls with HOST buffers: the library stages them through its own pinned/device
 * buffers (H2D + kernel + D2H on `stream`, synchronised before returning). These are what a
 * CPU-tensor caller of the binding reaches (rpu_base_tiles.cpp:405-445, 541-598). */
int ab200_tile_forward_host(ab200_tile *tile, const float *x_host, float *d_host, int bias,
                            int m_batch, int x_trans, int d_trans, int is_test, void *stream);
int ab200_tile_backward_host(ab200_tile *tile, const float *d_host, float *x_host, int bias,
                             int m_batch, int d_trans, int x_trans, void *stream);
int ab200_tile_update_host(ab200_tile *tile, const float *x_host, const float *d_host, int bias,
                           int m_batch, int x_trans, int d_trans, void *stream);

/* Signed coincidence counts of ONE sample for the deterministic pulse types
 * (DenseBitLineMaker::makeCoincidences, src/rpucuda/dense_bit_line_maker.cpp:266-331):
 * counts_dev is int32 [d_size][x_size]; positive count = weight decreases. Uses the tile's
 * update parameters, learning rate and weight granularity; weights are not touched. */
int ab200_tile_coincidences(ab200_tile *tile, const float *x_dev, const float *d_dev,
                            int32_t *counts_dev, void *stream);

/* ---- indexed (im2col-free) convolution interface -------------------------------------------
 * Replaces RPUSimple<T>::setMatrixIndices / hasMatrixIndices / forwardIndexed / backwardIndexed /
 * updateIndexed (src/rpucuda/rpu.h:452-478, src/rpucuda/rpu.cpp:846-1013, 1117-1239) as bound by
 * set_matrix_indices / forward_indexed / backward_indexed / update_indexed
 * (src/aihwkit/simulator/rpu_base_src/rpu_base_tiles_cuda.cpp:399-522, rpu_base_tiles.cpp:700-760).
 *
 * `indices` holds x_size * m_batch int32 entries, [x_size][m_batch] when `trans` is non-zero (the
 * layout AnalogConv2d builds, src/aihwkit/nn/modules/conv.py:534-571) or [m_batch][x_size]
 * otherwise: 0 = zero padding, 1 = the constant 1.0 (analog bias), j >= 2 = element j - 2 of an
 * image. It may be host or device memory and is copied (the reference borrows the pointer).
 * Images: x is [dim3][total_size / dim3]; d is [dim3][d_size][m_batch] when `trans`, else
 * [dim3][m_batch][d_size]. m_batch = output positions per image, dim3 = images per call (the
 * binding passes the batch size N and trans = 1). backward_indexed overwrites x_dev: every image
 * element is the sum, in ascending order of their position in the index array, of the input
 * gradients of the entries that name it (no atomics: the result is the same on every run).
 * Negative indices are rejected when the array is
 * set; an index beyond the image size is rejected by every call. */
int ab200_tile_set_matrix_indices(ab200_tile *tile, const int32_t *indices, long long count,
                                  void *stream);
int ab200_tile_has_matrix_indices(ab200_tile *tile);
int ab200_tile_forward_indexed(ab200_tile *tile, const float *x_dev, float *d_dev,
                               long long total_input_size, int m_batch, int dim3, int trans,
                               int is_test, void *stream);
int ab200_tile_backward_indexed(ab200_tile *tile, const float *d_dev, float *x_dev,
                                long long total_output_size, int m_batch, int dim3, int trans,
                                void *stream);
int ab200_tile_update_indexed(ab200_tile *tile, const float *x_dev, const float *d_dev,
                              long long total_input_size, int m_batch, int dim3, int trans,
                              void *stream);

/* ---- extra state (checkpoint / resume) ---------------------------------------------------------
 * Replaces RPUSimple / RPUPulsed / TransferRPUDevice::dumpExtra and loadExtra (src/rpucuda/rpu.cpp:
 * 405-503, rpu_pulsed.cpp:433-456, rpu_transfer_device.cpp:674-707) as bound by dump_extra /
 * load_extra (rpu_base_tiles.cpp:775-800): everything a resumed tile needs besides its weights and
 * hidden parameters, as name -> value pairs: learning rate, the Tiki-Taka update and column
 * counters and - unlike the reference, which does not save RNG state - the noise key and call
 * counters, so that a resumed run continues the same noise streams. `values` holds
 * ab200_tile_extra_count() doubles in the order of ab200_tile_extra_name(k). With `strict`
 * unknown or missing keys are errors. */
int ab200_tile_extra_count(void);
const char *ab200_tile_extra_name(int k);
int ab200_tile_dump_extra(ab200_tile *tile, double *values);
int ab200_tile_load_extra(ab200_tile *tile, const char *const *names, const double *values,
                          int count, int strict);
/* Vector-valued extra state: the choppers of the chopped / dynamic transfer compounds
 * ("rpu_device.in_chopper" [x_size], "rpu_device.out_chopper" [d_size], and for the dynamic form
 * "rpu_device.in_chopper_switched" [x_size]; in_chopper_ / out_chopper_ / in_chopper_switched_
 * of the reference's dumpExtra). count = 0 for every other device. Values are 0 or 1. */
int ab200_tile_extra_vector_count(const ab200_tile *tile);
const char *ab200_tile_extra_vector_name(const ab200_tile *tile, int k);
int ab200_tile_extra_vector_size(const ab200_tile *tile, int k);
int ab200_tile_get_extra_vector(ab200_tile *tile, int k, double *out);
int ab200_tile_set_extra_vector(ab200_tile *tile, int k, const double *in, int n);

/* Per-line values of a direction's IO (MVParameter, src/rpucuda/rpu_forward_backward_pass.h:14-22;
 * part of the reference's extra state as fwd.v_offset / fwd.out_nonlinearity / fwd.out_noise_values
 * and bwd.*, rpu_forward_backward_pass.cpp:66-79): `n` host floats, n = d_size forward, x_size
 * backward. Fails when the IO setting that uses the vector is off. */
enum ab200_io_vector {
  AB200_IOVEC_V_OFFSET = 0,
  AB200_IOVEC_OUT_NONLINEARITY = 1,
  AB200_IOVEC_OUT_NOISE_VALUES = 2
};
int ab200_tile_get_io_vector(ab200_tile *tile, int backward, int which, float *values_host, int n);
int ab200_tile_set_io_vector(ab200_tile *tile, int backward, int which, const float *values_host,
                             int n);

/* WeightModifierParameter (src/rpucuda/weight_modifier.h:15-50; bound in rpu_base_tiles.cpp:31-51). */
enum ab200_weight_modifier_type {
  AB200_WMOD_COPY = 0,
  AB200_WMOD_DISCRETIZE = 1,
  AB200_WMOD_MULT_NORMAL = 2,
  AB200_WMOD_ADD_NORMAL = 3,
  AB200_WMOD_DISCRETIZE_ADD_NORMAL = 4,
  AB200_WMOD_DOREFA = 5,
  AB200_WMOD_POLY = 6,
  AB200_WMOD_PCM_NOISE = 7, /* not implemented (nor by the reference's CPU tile) */
  AB200_WMOD_DROP_CONNECT = 8,
  AB200_WMOD_PROG_NOISE = 9
};
#define AB200_WMOD_MAX_COEFFS 8
typedef struct ab200_weight_modifier_params {
  int32_t type; /* enum ab200_weight_modifier_type */
  int32_t sto_round;
  int32_t enable_during_test;
  int32_t copy_last_column;
  int32_t rel_to_actual_wmax;
  int32_t n_coeffs;
  float std_dev;
  float res;
  float dorefa_clip;
  float pdrop;
  float assumed_wmax;
  float g_max;
  float coeffs[AB200_WMOD_MAX_COEFFS];
} ab200_weight_modifier_params;

/* RPUSimple::modifyFBWeights (src/rpucuda/rpu.cpp:1749-1758; WeightModifier::apply,
 * weight_modifier.cpp:31-215; rpu_base_tiles.cpp:358-371): forward and backward read a modified
 * copy of the weights from now on - discretised, with Gaussian noise relative to the largest
 * weight, DoReFa-quantised, with dropped connections ... - while updates keep going to the weights
 * themselves; the copy is refreshed by the next call. A forward with is_test != 0 reads the
 * weights themselves unless enable_during_test is set (RPUSimple::getFBWeights, rpu.cpp:1483-1487). */
int ab200_tile_modify_weights(ab200_tile *tile, const ab200_weight_modifier_params *params,
                              void *stream);

/* Power-law drift of the weights since they were last written (RPUPulsed::driftWeights,
 * src/rpucuda/rpu_pulsed.cpp:226-229; RPUSimple::driftWeights, rpu.cpp:1581-1587; WeightDrifter::
 * apply, weight_drifter.cpp:111-157; rpu_base_tiles.cpp:294-314). Elements whose weight changed by
 * more than reset_tol since the previous call restart their clock; the others are overwritten by
 * w0 * dt^(-nu) (plus the conductance-offset term), dt in units of t0 and at least 1. Pulsed
 * devices then clip to their bounds. The first call starts all clocks at zero. Not available for
 * Transfer compounds. */
int ab200_tile_drift_weights(ab200_tile *tile, float time_since_last_call, void *stream);

/* ---- weight operations between updates -------------------------------------------------------
 * Replace RPUPulsed<T>::decayWeights(alpha, bias_no_decay) / diffuseWeights() / clipWeights(...) /
 * resetCols(start_col, n_cols, reset_prob) / setWeightsUniformRandom (src/rpucuda/rpu_pulsed.cpp:
 * 189-282) with the per-element device rules of PulsedRPUDevice (src/rpucuda/rpu_pulsed_device.cpp:
 * 362-490), and for the floating-point (ideal) device the RPUSimple rules (src/rpucuda/rpu.cpp:
 * 1556-1625) and WeightClipper::apply (src/rpucuda/weight_clipper.cpp:38-118); bound as
 * decay_weights / diffuse_weights / clip_weights / reset_columns / set_weights_uniform_random
 * (rpu_base_tiles.cpp:263-400). All run on `stream` on the tile's weights in place. Compound
 * (Transfer) devices are not supported. */
enum ab200_clip_type {
  AB200_CLIP_NONE = 0,
  AB200_CLIP_FIXED_VALUE = 1,
  AB200_CLIP_LAYER_GAUSSIAN = 2,
  AB200_CLIP_AVERAGE_CHANNEL_MAX = 3
};
int ab200_tile_decay_weights(ab200_tile *tile, float alpha, int bias_no_decay, void *stream);
int ab200_tile_diffuse_weights(ab200_tile *tile, void *stream);
int ab200_tile_clip_weights(ab200_tile *tile, int clip_type, float fixed_value, float sigma,
                            void *stream);
int ab200_tile_reset_columns(ab200_tile *tile, int start_col, int n_cols, float reset_prob,
                             void *stream);
int ab200_tile_set_weights_uniform_random(ab200_tile *tile, float min_value, float max_value,
                                          void *stream);

/* Bound-management statistics of the last forward: number of samples that were re-run at least
 * once and the largest reduction factor used (rpu_forward_backward_pass.cpp:935-983). */
int ab200_tile_last_bm_stats(ab200_tile *tile, int32_t *n_rerun_samples, float *max_reduction);
/* Pulse counters of a device created with count_pulses (getPulseCounters, src/rpucuda/rpu.h:511;
 * get_pulse_counters, rpu_base_tiles.cpp:846-868): pulses that raised the weight in
 * out[0][d][x], pulses that lowered it in out[1][d][x], summed over all updates since the tile
 * was made (a pulse counts whether or not the weight was at its bound). `out` holds
 * 2 * d_size * x_size values, row-major [2][d_size][x_size] (the reference hands out its device
 * layout unchanged). Returns an error if the device does not count. */
int ab200_tile_get_pulse_counters(ab200_tile *tile, int64_t *out_host);
int ab200_tile_counts_pulses(ab200_tile *tile);

/* Re-key the noise generator (RPUSimple::setRandomSeed, src/rpucuda/rpu.cpp:1516-1520). */
int ab200_tile_set_seed(ab200_tile *tile, uint64_t seed);

/* ---- mapped-tile layer ----------------------------------------------------------------- */

/* A logical [out_size][in_size] layer split into physical tiles of at most
 * max_output_size x max_input_size (TileModuleArray, src/aihwkit/simulator/tiles/array.py:43-198;
 * split rule get_split_sizes :82-97). All tiles share `cfg` (x_size/d_size in cfg are ignored).
 * Only the in-splits [in_split_begin, in_split_end) are materialised on this GPU, which is how a
 * rank of a sharded layer owns its share; pass 0 and the total number of in-splits (or -1) for
 * the whole layer. */
int ab200_array_create(const ab200_tile_config *cfg, int out_size, int in_size,
                       int max_output_size, int max_input_size, int in_split_begin,
                       int in_split_end, int cuda_device, ab200_array **out);
/* The same for a block of the layer's tiles, in-splits [in_split_begin, in_split_end) x
 * out-splits [out_split_begin, out_split_end) (an end of -1 = to the last): the 2-D tile -> GPU
 * map of a layer with fewer in-splits than ranks. Forward writes the block's columns of y and
 * zeroes the others, so that the shards' results add up; the digital bias is added by the
 * shards that hold in-split 0; noise streams are those of the tile's place in the whole layer. */
int ab200_array_create_block(const ab200_tile_config *cfg, int out_size, int in_size,
                             int max_output_size, int max_input_size, int in_split_begin,
                             int in_split_end, int out_split_begin, int out_split_end,
                             int cuda_device, ab200_array **out);
int ab200_array_destroy(ab200_array *arr);
int ab200_array_num_in_splits(const ab200_array *arr);
int ab200_array_num_out_splits(const ab200_array *arr);
/* Host [out_size][in_size] logical weights (TileModuleArray.set_weights, array.py:112-135);
 * only the locally owned in-splits are read / written. */
int ab200_array_set_weights(ab200_array *arr, const float *w_host);
int ab200_array_get_weights(ab200_array *arr, float *w_host);
/* Digital periphery of the mapped layer, applied inside the layer's kernels.
 * set_weights_scaled: as set_weights, but every tile's weights are divided by
 * alpha = max|w_tile| / omega and alpha becomes that tile's digital output scale
 * (TileWithPeriphery.apply_weight_scaling / set_scales, layer-wise form,
 * src/aihwkit/simulator/tiles/periphery.py:437-500, 689-728; forward: apply_out_scaling :785-805).
 * omega <= 0 means no scaling. get_weights returns the logical (re-scaled) weights.
 * get_tile_scales: the scales of the locally owned tiles, [local in-splits][out-splits].
 * set_bias: digital bias [out_size] added once after the sum over in-splits (array.py:178-181);
 * NULL removes it. On a sharded layer only one rank should hold the bias. */
/* Training of a mapped layer, tile by tile as autograd drives the tiles of TileModuleArray in the
 * reference (TileWithPeriphery.pre_backward / backward / pre_update / update,
 * src/aihwkit/simulator/tiles/periphery.py:1068-1110, 1154-1230): backward writes
 * x_grad[:, in-split i] = sum over out-splits o of tile(i, o).backward(d[:, out-split o] *
 * alpha_io); update runs tile(i, o).update(x[:, in-split i], d[:, out-split o] / alpha_io).
 * d_dev is [m_batch][out_size]; x_dev / x_grad_dev are [m_batch][in_size]; only the locally owned
 * input columns are read / written. */
int ab200_array_backward(ab200_array *arr, const float *d_dev, float *x_grad_dev, int m_batch,
                         void *stream);
int ab200_array_update(ab200_array *arr, const float *x_dev, const float *d_dev, int m_batch,
                       void *stream);
int ab200_array_set_learning_rate(ab200_array *arr, float lr);
int ab200_array_set_weights_scaled(ab200_array *arr, const float *w_host, float omega);

/* ---- sharded layer: partial sums pushed to the row-block owners (no counterpart in the
 * reference, which has no multi-GPU path) ----------------------------------------------------
 * ab200_array_forward_scatter: forward of this rank's tiles on its own input columns
 * x_local_dev [m_batch][local_in_size]; instead of one local [m_batch][out_size] partial sum, the
 * rows are written straight into the buffers of their owners: row r goes to
 * out_table_dev[r / rows_per_owner] at row r % rows_per_owner, row pitch out_size. out_table_dev
 * is a DEVICE array of n_owners pointers; the pointers may be peer memory opened with
 * ab200_peer_open (plain stores over NVLink, no multicast). rotate_rows is the row this rank's
 * sweep over the row blocks starts at. Needs the tensor-core path.
 * ab200_sum_slots: out[e] = sum over k < n_slots of slots[k * elems + e]: the owner adds the
 * partial sums the ranks wrote side by side (call it after a barrier over the ranks).
 * ab200_peer_*: cudaMalloc'ed buffers shared between the processes of one node with CUDA IPC;
 * handle_out / handle are 64 opaque bytes to pass to the other ranks. */
int ab200_array_forward_scatter(ab200_array *arr, const float *x_local_dev, int m_batch,
                                float *const *out_table_dev, int n_owners, int rows_per_owner,
                                int rotate_rows, void *stream);
int ab200_sum_slots(const float *slots_dev, int n_slots, long long elems, float *out_dev,
                    void *stream);
/* The same with a quarter (or less) of the bytes on the wire, for layers whose ADC codes fit a
 * signed byte (ab200_array_scatter_codes_supported: noisy inference settings, no bound management,
 * out-splits that are multiples of 128, no mapping scales / bias on this array): the kernel sends
 * the integer ADC code of every in-split instead of the fp32 sum over the rank's in-splits.
 * code_table_dev[owner] points to this rank's slot at the owner: n_in_splits planes of
 * rows_per_owner x out_size bytes, each plane in blocks of 32 rows x 32 columns (1 KB, row-major,
 * blocks ordered by row block, then column block); fac_table_dev[owner] to
 * [n_in_splits][rows_per_owner] floats (the factor of each row and in-split).
 * ab200_sum_code_slots: the owner's sum out[r][c] = sum over slots q (in order) of
 * (sum over planes i < n_planes[q] of code * factor), the same association as the fp32 variant;
 * slot q starts at code_slots_dev + q * code_slot_stride (bytes) and fac_slots_dev + q *
 * fac_slot_stride (floats); rows_valid <= rows_per_owner rows are written. */
int ab200_array_scatter_codes_supported(ab200_array *arr);
int ab200_array_forward_scatter_codes(ab200_array *arr, const float *x_local_dev, int m_batch,
                                      unsigned char *const *code_table_dev,
                                      float *const *fac_table_dev, int n_owners,
                                      int rows_per_owner, int rotate_rows, void *stream);
int ab200_sum_code_slots(const unsigned char *code_slots_dev, long long code_slot_stride,
                         const float *fac_slots_dev, long long fac_slot_stride, int n_slots,
                         const int *n_planes, int rows_per_owner, int rows_valid, int out_size,
                         float *out_dev, void *stream);
/* General form of the two scatter calls above, for a batch that is cut into several launches, for
 * rows dealt to the owners in blocks, and for owners that learn of the arrival from a flag
 * instead of a barrier over the ranks (no counterpart in the reference):
 *  - row_base: row of the whole batch this launch starts at (a multiple of 32); noise draws and
 *    owners are those of the row of the whole batch, so cutting a batch does not change where a
 *    row goes.
 *  - owner_block_rows = 0: owner q holds the rows [q * rows_per_owner, (q + 1) * rows_per_owner).
 *    owner_block_rows = B > 0 (a multiple of 32): block b = row / B of the batch is block
 *    b / n_owners of owner b % n_owners, so that every part of a batch in row order feeds all
 *    owners alike. rows_per_owner is the number of rows an owner's buffer holds either way.
 *  - flag_table_dev (or null): device array of n_owners addresses, local or peer memory; when
 *    every store of the launch has been issued and fenced at system scope, the kernel writes
 *    `epoch` to each of them. Epochs of successive launches must increase.
 * Exactly one of out_table_dev and code_table_dev (+ fac_table_dev) is given.
 * ab200_sum_slots_wait / ab200_sum_code_slots_wait: the owner's side. The kernel first waits until
 * all n_flags words at flags_dev (this owner's arrival flags, one per sender) have reached
 * `epoch` - at most max_wait_ms, then it gives up WITHOUT summing, records the failure, and the
 * next ab200_wait_status call (after synchronising the stream) reports it - then adds the slots
 * for the local rows [row0, row0 + rows): out[r][c] = sum over k of slots[k * slot_stride + r *
 * out_size + c] (slot_stride in floats). The waiting kernel and the kernels that raise the flags
 * must run on different GPUs (or the flags must already be up): kernels of one GPU do not
 * necessarily run at the same time.
 * ab200_wait_status: 0, or the number of waits that ran out since the last call (and clears it). */
typedef struct ab200_scatter_plan {
  float *const *out_table_dev;
  unsigned char *const *code_table_dev;
  float *const *fac_table_dev;
  int32_t *const *flag_table_dev;
  int32_t n_owners;
  int32_t rows_per_owner;
  int32_t rotate_rows;
  int32_t row_base;
  int32_t owner_block_rows;
  int32_t epoch;
} ab200_scatter_plan;
int ab200_array_forward_scatter_plan(ab200_array *arr, const float *x_local_dev, int m_batch,
                                     const ab200_scatter_plan *plan, void *stream);
int ab200_sum_slots_wait(const float *slots_dev, int n_slots, long long slot_stride, int row0,
                         int rows, int out_size, float *out_dev, const int32_t *flags_dev,
                         int n_flags, int epoch, float max_wait_ms, void *stream);
int ab200_sum_code_slots_wait(const unsigned char *code_slots_dev, long long code_slot_stride,
                              const float *fac_slots_dev, long long fac_slot_stride, int n_slots,
                              const int *n_planes, int rows_per_owner, int row0, int rows,
                              int out_size, float *out_dev, const int32_t *flags_dev, int n_flags,
                              int epoch, float max_wait_ms, void *stream);
int ab200_wait_status(int cuda_device, int *timed_out);
int ab200_peer_alloc(size_t bytes, int cuda_device, void **dev_ptr, unsigned char handle_out[64]);
int ab200_peer_open(const unsigned char handle[64], int cuda_device, void **dev_ptr);
int ab200_peer_close(void *dev_ptr);
int ab200_peer_free(void *dev_ptr);
int ab200_array_get_tile_scales(ab200_array *arr, float *scales_host);
int ab200_array_set_bias(ab200_array *arr, const float *bias_host);
/* TileModuleArray.forward (array.py:155-182): every tile does its own noise management, DAC,
 * MVM and ADC; results of the in-splits are added after the ADC, out-splits are concatenated.
 * x_dev is the full [m_batch][in_size] input; y_dev is [m_batch][out_size] and receives the sum
 * over the locally owned in-splits (the partial sum a sharded rank contributes). */
int ab200_array_forward(ab200_array *arr, const float *x_dev, float *y_dev, int m_batch,
                        int is_test, void *stream);
int ab200_array_forward_host(ab200_array *arr, const float *x_host, float *y_host, int m_batch,
                             int is_test, void *stream);
/* Same as ab200_array_forward for a rank of a sharded layer whose input holds only the columns
 * of its own in-splits: x_local_dev is [m_batch][ab200_array_local_in_size()] (the reference
 * passes each in-split its slice of the input, array.py:165-167). */
int ab200_array_forward_local(ab200_array *arr, const float *x_local_dev, float *y_dev,
                              int m_batch, int is_test, void *stream);
int ab200_array_local_in_size(const ab200_array *arr);
int ab200_array_set_seed(ab200_array *arr, uint64_t seed);

/* ---- forward pass without any allocation ------------------------------------------------- */

/* No counterpart in the reference (its GPU tile allocates buffers on demand).
 *
 * For hosts that pre-reserve the GPU's memory and forbid allocation afterwards - an inference
 * server's execute callback, a real-time loop, a plugin with a "no allocation after init"
 * contract - where a cudaMalloc mid-request would fail or stall every stream of the device.
 * Computes the IO-managed forward pass of ab200_tile_forward (non-transposed layouts, no bias)
 * from caller-owned memory only: w_dev_xd is the fp32 [x_size][d_size] weight, x_dev is
 * [m_batch][x_size], d_dev is [m_batch][d_size]. It always runs the CUDA-core kernels (the
 * tensor-core path keeps an operand copy of the weights that it would have to allocate), so for
 * sizes where ab200_tile_forward picks the tensor cores the two agree up to the summation order:
 * a rare element may land on the neighbouring ADC step. All pointers belong to the CURRENT CUDA
 * device of the calling thread, which is also the device whose scratch array is used: make the
 * device current (cudaSetDevice) before the call. The per-sample scratch lives in a fixed array
 * inside the library image (about 320 KB per GPU, held until the process exits), so m_batch is
 * limited to AB200_NOALLOC_MAX_BATCH; larger batches are rejected with an error - split them.
 * The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *  - The first call on each device looks up the array's device address; make that first call
 *    during start-up, outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's contents (the
 *    library clears what has to start at zero): calls that overlap on the GPU - different
 *    streams, or several host threads - race on it. Run them one after the other.
 *  - (seed, call) key the noise: the same pair reproduces the same noise; vary `call`. */
#define AB200_NOALLOC_MAX_BATCH 16384
int ab200_mvm_forward_noalloc(const ab200_io_params *forward_io, const float *w_dev_xd,
                              int x_size, int d_size, const float *x_dev, float *d_dev,
                              int m_batch, uint64_t seed, uint32_t call, void *stream);

/* Kernel selection for the MVM (no counterpart in the reference, which always calls cuBLAS):
 * 0 = automatic (tensor cores for large aligned problems), 1 = CUDA cores only, 2 = tensor
 * cores whenever the IO settings allow, 3 = as 2 but never the kernel variant that pairs two
 * CTAs on one 256-row tile. Process-wide; used by tests and benchmarks. */
int ab200_set_mvm_path(int mode);
/* Kernel selection of the pulsed update, for tests and benchmarks: 0 = automatic (stochastic pulse
 * trains with batches of 1024 samples or more stream over the samples of each x-line, everything
 * else goes through the kernel that stages blocks of samples per weight tile), 1 = always the
 * staged kernel, 2 = the streaming kernel for every batch size the pulse type allows. */
int ab200_set_update_path(int mode);
/* Measurement aid (no counterpart in the reference): AND + population count + add triples per
 * second the device sustains from registers, the integer ceiling that the pair rate of the pulsed
 * update at large batches (x_size * d_size * m_batch word pairs per call) is compared with. */
int ab200_measure_popc_peak(int cuda_device, double *pairs_per_s);

/* Number of kernels this library has launched since it was loaded (all tiles, this process). */
uint64_t ab200_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* AIHWKIT_B200_H_ */
