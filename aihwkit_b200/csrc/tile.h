// Host-side analog tile: the B200 counterpart of RPUSimple / RPUPulsed
// (src/rpucuda/rpu.h:194-706, src/rpucuda/rpu_pulsed.h:23-125) for the hot path.
#pragma once

#include "../../include/aihwkit_b200.h"
#include "common.cuh"

#include <cuda_runtime.h>

#include <memory>
#include <mutex>
#include <string>
#include <random>
#include <vector>

namespace ab200 {

// IOMetaParameter after initializeForForward / initializeForBackward
// (src/rpucuda/rpu_pulsed_meta_parameter.cpp:40-128): resolutions already multiplied by
// 2 * bound, infinite bounds resolved.
struct IOEff {
  int is_perfect;
  int nm; // ab200_noise_management
  int bm; // ab200_bound_management
  int w_noise_type;
  int bm_test_negative_bound;
  int max_bm_factor;
  float max_bm_res;
  float inp_bound;
  float res_in;
  float out_bound;
  float res_out;
  float out_noise;
  float out_noise_std; // > 0: the kernels read the std-dev of every output line from a table
  float out_scale;
  float w_noise;
  float nm_thres;
  float nm_assumed_wmax;
  float nm_decay; // running-average noise management
  // non-idealities of the output lines (CUDA-core kernels): IR drop, voltage offsets / series
  // resistance, output non-linearity; the per-line tables travel in MvmProblem
  float ir_drop;
  float ir_g_ratio;
  float v_offset_std;
  float r_series;
  float r_series_max;
  float out_nl, out_nl_std, slope_calibration;
  // Gaussian added to the DAC output, factors applied to negative DAC outputs / negative values
  // in front of the ADC (1 - asymmetry), stochastic rounding of DAC / ADC
  float inp_noise;
  float inp_asym;
  float out_asym;
  int inp_sto_round;
  int out_sto_round;
  // 0: one pass; 1 / 2: negative and positive inputs in two passes, summed before / after the
  // output stage (CUDA-core kernels)
  int pos_neg;
};

// `plain_only`: reject the settings only the forward / backward kernels implement (input noise,
// asymmetries, stochastic rounding), as for the read-out of a transfer.
IOEff resolveIO(const ab200_io_params &io, bool backward, bool plain_only = false);

// PulsedUpdateMetaParameter after initialize() (rpu_pulsed_meta_parameter.cpp:134-151).
constexpr int kPulseSegSlots = 31; // pulse slots of one 32-bit pulse word (bit 0 is the sign)

struct UpEff {
  int pulse_type;
  int desired_bl;
  int fixed_bl;
  int update_management;
  int update_bl_management;
  int sto_round; // stochastic rounding of the pulse probabilities to `res`
  float um_grad_scale;
  float res;
  float x_res_implicit;
  float d_res_implicit;
};

UpEff resolveUp(const ab200_update_params &up);

// One IO-managed matrix-vector batch: out[s][n] = IO( sum_k in[s][k] * W(k, n) ).
// Rows read through the index array of the indexed convolution interface instead of from a
// matrix: row r is output position l = r % m_batch of image n = r / m_batch, its element k is
// element idx[l * ld + k] - 2 of that image (entry 0: padding, reads as 0; entry 1: the constant
// input of an analog bias, reads as 1). `idx` is null for plain rows.
struct RowGather {
  const int32_t *idx = nullptr; // [m_batch][ld]
  int m_batch = 0;
  int ld = 0;
  long long image_size = 0; // elements between two images
};

struct MvmProblem {
  const float *in;
  long long in_ss, in_fs; // strides of sample / feature
  int in_size;            // K (including an appended bias feature)
  int in_real;            // features k >= in_real read as 1.0 (bias column)
  float *out;
  long long out_ss, out_fs;
  int out_size;  // N
  int out_store; // only n < out_store is written
  int accumulate; // add to `out` instead of overwriting it
  const float *w;
  long long wk, wn; // W(k, n) = w[k * wk + n * wn]
  int m;
  int backward;
  IOEff io;
  float alpha; // fwd / bwd alpha scale of the tile (1 unless set)
  PhiloxKey key;
  uint32_t call;
  uint32_t noise_id; // distinguishes tiles of a mapped array in the noise counter
  // per-sample scratch (m entries each)
  float *scale;  // input scale; 0 marks a row whose output is identically zero
  float *factor; // output factor
  float *vnorm;  // || prepared input ||_2 (only when weight noise is on)
  float *sval;   // noise-management value s
  int *flags;    // bound management: sample clipped in round 1
  int *bm_stats; // [0] re-run samples, [1] max reduction (float bits)
  // std-dev of the output noise of every output line (out_size entries) when io.out_noise_std > 0
  const float *out_noise_vals = nullptr;
  // running value of the AverageAbsMax noise management (one float, < 0: not started), shared by
  // the forward and backward passes of a tile as in the reference
  float *nm_state = nullptr;
  // per-line voltage offsets and output non-linearities (out_size entries each) and the slope
  // calibration factor, when the IO of this direction has them
  const float *v_offset = nullptr;
  const float *out_nl = nullptr;
  float nl_factor = 1.0f;
  // tensor-core path only: `in` holds whole images and the rows are gathered from them
  RowGather gather;
  // > 0: outputs stored transposed in blocks of that many rows, row r / column n at
  // out[((r / out_t_rows) * out_size + n) * out_t_rows + r % out_t_rows] (out_ss / out_fs unused)
  int out_t_rows = 0;
};

// CUDA-core path: noise management, fused MVM, bound-management re-run
void launchMvm(const MvmProblem &p, cudaStream_t stream);
// bound-management re-run of the rows whose first round clipped (forward only; no-op otherwise)
void launchBmRerun(const MvmProblem &p, cudaStream_t stream);

// Kernel selection for the MVM: 0 = automatic, 1 = always CUDA cores, 2 = tensor cores whenever
// the problem can be expressed on them.
void setMvmPath(int mode);
int mvmPath();

// Per-element device parameters in the update kernel's layout, index = x * d_size + d.
struct DeviceStore {
  int kind = AB200_DEVICE_IDEAL;
  float dw_min = 0.001f;
  float dw_min_std = 0.0f;
  int mult_noise = 1;
  float4 *par4 = nullptr; // {scale_up, scale_down, max_bound, min_bound}
  float2 *par2 = nullptr; // {slope_up, slope_down} or {reference, 0}
  float4 *par3 = nullptr; // {decay_scale, diffusion_rate, reset_bias, 0}; uploaded on first use
  bool par3_valid = false;
  float reset_std = 0.0f;
  // ExpStep: {a, b, A_up, A_down} and {gamma_up, gamma_down, dw_min_std_add, dw_min_std_slope}
  float4 es0 = {0.f, 0.f, 0.f, 0.f}, es1 = {0.f, 0.f, 0.f, 0.f};
  // PiecewiseStep: pw_n factors for the up direction followed by pw_n for the down direction
  std::vector<float> pw_host;
  float *pw = nullptr;
  int pw_n = 0;
  // host copies, [name][d][x] in the reference's naming / order
  std::vector<std::string> names;
  std::vector<float> host;
};

struct UpdateProblem {
  const float *x;
  long long x_ss, x_fs;
  int x_real; // features >= x_real read as 1.0 (bias)
  const float *d;
  long long d_ss, d_fs;
  int x_size, d_size, m;
  // Stochastic pulse trains longer than 31 slots are cut into segments of at most 31: a sample
  // then has `nseg` rows of pulse words (row = sample * nseg + segment), each with its own sign
  // bit, and the update kernels see m * nseg rows. Coincidences of one sample commute, so the
  // per-weight result is that of the reference's multi-word trains
  // (nK32 words per line, src/rpucuda/cuda/bit_line_maker.cu:24-28).
  int nseg;
  float lr;     // |pulse-count learning rate|
  int lr_neg;   // learning rate negative
  float dw_min; // weight granularity
  UpEff up;
  PhiloxKey key;
  uint32_t call;
  // scratch
  uint32_t *xw; // [m][x_size] pulse words (or float bit patterns for implicit pulses)
  uint32_t *dw; // [m][d_size]
  // target
  float *w;
  const float4 *par4;
  const float2 *par2;
  int kind;
  float dw_min_std;
  int mult_noise;
  float4 es0, es1; // ExpStep globals (DeviceStore)
  const float *pw;  // PiecewiseStep tables (DeviceStore), pw_n nodes per direction
  int pw_n;
  // choppers of a chopped transfer compound (one byte per x-line / d-line, non-zero = the sign
  // of that line's pulses is flipped), or null
  const unsigned char *chop_x, *chop_d;
  int s_begin, s_end; // sample range applied by the update kernel
  // pulsed update only: `x` holds whole images and the samples are gathered from them
  RowGather gather;
};

void launchPulsePrepare(const UpdateProblem &p, cudaStream_t stream);
// Stochastic pulse trains: the update streams over the non-empty samples of an x-line (transposed
// x words, their bitmaps and compacted lists) instead of staging blocks of samples per weight
// tile. Measured faster from a batch of 64 (256 x 256 tile) upwards; below one bitmap word of
// samples the three extra launches are not worth it.
constexpr int kStreamUpdateMinBatch = 32;
bool streamUpdateEligible(const UpdateProblem &p);
// kernel selection of the pulsed update: 0 = automatic, 1 = always the staged kernel, 2 = the
// streaming kernel whenever the pulse type allows it (any batch size)
void setUpdatePath(int mode);
void launchPulseTranspose(const UpdateProblem &p, uint32_t *xwT, uint32_t *xnzT, int m_pad,
                          cudaStream_t stream);
// compacted (sample, word) lists of every x-line, from the transposed words and their bitmaps
void launchPulseCompact(const UpdateProblem &p, const uint32_t *xwT, const uint32_t *xnzT, int m_pad,
                        uint32_t *list_s, uint32_t *list_x, uint32_t *list_off, cudaStream_t stream);
void launchPulsedUpdateStream(const UpdateProblem &p, const uint32_t *xwT, const uint32_t *xnzT,
                              int m_pad, cudaStream_t stream, const uint32_t *list_s,
                              const uint32_t *list_x, const uint32_t *list_off);
void launchPulsedUpdate(const UpdateProblem &p, cudaStream_t stream);
void launchCoincidences(const UpdateProblem &p, int32_t *counts_dx, cudaStream_t stream);
// pulses of the samples [s_begin, s_end) of a prepared batch, added per weight to `up` (the weight
// rises) and `down` (it falls), both [x][d]
void launchPulseCounter(const UpdateProblem &p, unsigned long long *up, unsigned long long *down,
                        cudaStream_t stream);
void launchFPUpdate(const UpdateProblem &p, float lr_signed, cudaStream_t stream,
                    bool overwrite = false, bool clip_each = false);
// Chopped transfer: de-chop the read of column `col`, accumulate it in the buffer column in units
// of the buffer granularity, turn whole units into the write-out (d = -n), flip the in chopper of
// the column when `flip_in` is set (ChoppedTransferRPUDevice::readAndUpdate,
// rpu_chopped_transfer_device.cpp:357-470)
void launchTransferChopBuffer(float *buffer_col, float *read_inout, int d_size, float lr_scale,
                              float max_steps, float momentum, int forget_buffer, int no_buffer,
                              unsigned char *chop_in, int col, const unsigned char *chop_out,
                              int flip_in, cudaStream_t stream);
// Dynamic transfer: as above, with the read taken against the reference mean of the element
// (replaced by its running mean when the in chopper of the line flipped at the previous
// transfer), the running mean advanced by the read, and the buffer clamped to +-buffer_cap
// (DynamicTransferRPUDevice::readAndUpdate, rpu_dynamic_transfer_device.cpp:198-343)
void launchTransferDynamicBuffer(float *buffer_col, float *mean_col, float *past_col,
                                 float *read_inout, int d_size, float lr_scale, float max_steps,
                                 float momentum, int forget_buffer, float buffer_cap,
                                 float sample_momentum, int previously_switched,
                                 unsigned char *chop_in, int col, const unsigned char *chop_out,
                                 int flip_in, cudaStream_t stream);
// Mixed-precision compound: quantised copies of the x / d samples of a batch; pulse counts (and
// one-hot d vectors) of the rows of chi that a transfer moves to the device
void launchMixedQuantize(const UpdateProblem &p, int n_x_bins, int n_d_bins, int sr_x, int sr_d, float *qx,
                         float *qd, cudaStream_t stream);
void launchMixedTruncate(float *chi, int x_size, int d_size, int row0, int n_rows, float gran, float *counts,
                         float *onehot, cudaStream_t stream);
// flip every out chopper with probability `prob`
void launchFlipChoppers(unsigned char *chop, int n, float prob, PhiloxKey key, uint32_t call,
                        cudaStream_t stream);
void launchTransferRead(const float *w_fast, int col, int d_size, const IOEff &io, PhiloxKey key,
                        uint32_t call, float *x_onehot, int x_size, float *r_out, float alpha,
                        cudaStream_t stream);
// buffered Transfer: accumulate a read-out column into the buffer, emit the whole steps
void launchTransferBuffer(float *buffer_col, float *read_inout, int d_size, float lr_abs,
                          float buffer_granularity, float max_steps, float momentum,
                          int forget_buffer, cudaStream_t stream);
void launchTransposeDX(const float *src, float *dst, int rows, int cols, cudaStream_t stream);
void launchClipToBounds(float *w, const float4 *par4, long long n, cudaStream_t stream);
// AND + popc + add triples per second the current device sustains from registers
double measurePopcPeak(cudaStream_t stream);
// dst[r * dst_ld + c] += src[r * src_ld + c]
void launchAddBlock(const float *src, long long src_ld, float *dst, long long dst_ld, int rows,
                    int cols, cudaStream_t stream);

class TcEngine;

class Tile {
public:
  Tile(const ab200_tile_config &cfg, int cuda_device);
  ~Tile();
  Tile(const Tile &) = delete;
  Tile &operator=(const Tile &) = delete;

  std::mutex &mutex() const { return mu_; }
  int xSize() const { return x_size_; }
  int dSize() const { return d_size_; }
  int device() const { return device_; }
  void toDevice(int cuda_device);

  void setLearningRate(float lr) { lr_ = lr; }
  float learningRate() const { return lr_; }
  void setSeed(uint64_t seed);

  void setWeights(const float *w_host_dx);
  void getWeights(float *w_host_dx);
  void setWeightsDevice(const float *w_dev_xd, cudaStream_t s);
  void getWeightsDevice(float *w_dev_xd, cudaStream_t s);
  void setSharedWeights(float *w_dev_xd, uint64_t version);
  // RPUSimple::setDeltaWeights (src/rpucuda/rpu.cpp:1459-1481): while set, the floating-point
  // update writes +sum_s d x / bwd_alpha into this [x][d] buffer and leaves the weights alone
  // (getAlphaLearningRate :1400-1403, getUpBeta :1509-1511); null = back to normal
  void setDeltaWeights(float *dw_dev_xd);

  int hiddenCount() const;
  const char *hiddenName(int i) const;
  void getHidden(float *out);
  void setHidden(const float *in);

  // out_t_rows > 0: the output is stored transposed in blocks of that many rows
  // (MvmProblem::out_t_rows); d_trans must be false then
  void forward(const float *x, float *d, bool bias, int m, bool x_trans, bool d_trans,
               bool is_test, cudaStream_t s, int out_t_rows = 0);
  void backward(const float *d, float *x, bool bias, int m, bool d_trans, bool x_trans,
                cudaStream_t s);
  void update(const float *x, const float *d, bool bias, int m, bool x_trans, bool d_trans,
              cudaStream_t s);
  void forwardHost(const float *x, float *d, bool bias, int m, bool x_trans, bool d_trans,
                   bool is_test, cudaStream_t s);
  void backwardHost(const float *d, float *x, bool bias, int m, bool d_trans, bool x_trans,
                    cudaStream_t s);
  void updateHost(const float *x, const float *d, bool bias, int m, bool x_trans, bool d_trans,
                  cudaStream_t s);
  void coincidences(const float *x, const float *d, int32_t *counts, cudaStream_t s);

  // indexed convolution interface (RPUSimple::setMatrixIndices / forwardIndexed / backwardIndexed /
  // updateIndexed, src/rpucuda/rpu.h:452-478); `indices` may be host or device memory and is copied
  void setMatrixIndices(const int32_t *indices, long long n, cudaStream_t s);
  bool hasMatrixIndices() const { return idx_count_ != 0; }
  void forwardIndexed(const float *x, float *d, long long total_input_size, int m_batch, int n_img,
                      bool trans, bool is_test, cudaStream_t s);
  void backwardIndexed(const float *d, float *x, long long total_output_size, int m_batch,
                       int n_img, bool trans, cudaStream_t s);
  void updateIndexed(const float *x, const float *d, long long total_input_size, int m_batch,
                     int n_img, bool trans, cudaStream_t s);
  void lastBmStats(int32_t *n_rerun, float *max_red);
  // vector-valued extra state (choppers of the chopped / dynamic transfer compounds)
  int extraVectorCount() const;
  const char *extraVectorName(int k) const;
  int extraVectorSize(int k) const;
  void getExtraVector(int k, double *out);
  void setExtraVector(int k, const double *in, int n);
  bool countsPulses() const { return cfg_.device[0].count_pulses != 0; }
  void getPulseCounters(int64_t *out_2dx);

  // state that is neither a weight nor a hidden parameter, as name -> value pairs
  // (RPUSimple / RPUPulsed / TransferRPUDevice::dumpExtra / loadExtra, src/rpucuda/rpu.cpp:405-503,
  // rpu_pulsed.cpp:433-456, rpu_transfer_device.cpp:674-707), plus the noise key and counters
  static int extraCount();
  static const char *extraName(int k);
  void dumpExtra(double *values) const;
  void loadExtra(const char *const *names, const double *values, int n, bool strict);

  // weight operations between updates (RPUPulsed::decayWeights / diffuseWeights / clipWeights /
  // resetCols / setWeightsUniformRandom, src/rpucuda/rpu_pulsed.cpp:189-284)
  void getIoVector(bool backward, int which, float *values, int n);
  void setIoVector(bool backward, int which, const float *values, int n);
  void driftWeights(float time_since_last_call, cudaStream_t s);
  void modifyWeights(const ab200_weight_modifier_params &par, cudaStream_t s);
  void decayWeights(float alpha, bool bias_no_decay, cudaStream_t s);
  void diffuseWeights(cudaStream_t s);
  void clipWeights(int type, float fixed_value, float sigma, cudaStream_t s);
  void resetColumns(int start_col, int n_cols, float reset_prob, cudaStream_t s);
  void setWeightsUniformRandom(float lo, float hi, cudaStream_t s);

  // used by the mapped array: forward on a sub-block of a wider activation matrix
  void forwardStrided(const float *x, long long x_ss, float *y, long long y_ss, int m,
                      bool accumulate, uint32_t noise_id, float out_scale, cudaStream_t s);

  void backwardStrided(const float *d, long long d_ss, float *x, long long x_ss, int m,
                       bool accumulate, uint32_t noise_id, float out_scale, cudaStream_t s);
  void updateStrided(const float *x, long long x_ss, const float *d, long long d_ss, int m,
                     cudaStream_t s);

  const IOEff &fio() const { return f_io_; }
  float *weightsXD() { return w_; }
  uint64_t weightsVersion() const { return w_version_; }
  PhiloxKey noiseKey() const { return key_; }
  uint32_t nextForwardCall() { return fwd_calls_++; }

private:
  void requireDevice(const char *what) const;
  void ensureScratch(int m);
  void ensureStage(size_t n_floats);
  void uploadDeviceStore(DeviceStore &ds);
  void populateHost();
  void fillMvmScratch(MvmProblem &p);
  bool tcEligible(const MvmProblem &p) const;
  void runTc(const MvmProblem &p, cudaStream_t s);
  void pulsedUpdateRange(UpdateProblem &p, cudaStream_t s);
  void doTransfer(cudaStream_t s);
  float pulseCountLR() const;
  void backwardCore(const float *d, long long d_ss, long long d_fs, float *x, long long x_ss,
                    long long x_fs, int x_store, int m, bool accumulate, uint32_t noise_id,
                    float out_scale, cudaStream_t s, int out_t_rows = 0);
  void updateCore(const float *x, long long x_ss, long long x_fs, int x_in, const float *d,
                  long long d_ss, long long d_fs, int m, cudaStream_t s);
  void requireSingleDevice(const char *what);
  void ensurePar3(DeviceStore &ds);
  int opTargets(float *w[2], DeviceStore *ds[2]);
  void requireIndices(const char *what, long long image_size, int m_batch, int n_img) const;
  void ensureIndexedScratch(long long b, bool need_x, bool need_d);
  // the index array as [m_batch][x_size] (transposed on the device when the caller's is
  // [x_size][m_batch])
  const int32_t *rowMajorIndices(int m_batch, bool trans, cudaStream_t s);
  // whether the forward pass / the update of `b` gathered rows can read the images directly
  bool forwardGatherEligible(int b) const;
  bool updateGatherEligible() const;
  void forwardGathered(const float *images, const RowGather &g, float *d, int b, bool is_test,
                       cudaStream_t s, int out_t_rows);
  void gatherIndexed(const float *x, long long in_mat, int m_batch, int n_img, bool trans,
                     cudaStream_t s);

  mutable std::mutex mu_; // held by every C-ABI call on this tile
  ab200_tile_config cfg_;
  int x_size_, d_size_;
  int device_ = -1;
  float lr_ = 0.1f; // createRPUArray sets 0.1 (rpu_pulsed.cpp:54)
  IOEff f_io_, b_io_, t_io_;
  UpEff up_, t_up_;
  PhiloxKey key_;
  uint32_t fwd_calls_ = 0, bwd_calls_ = 0, upd_calls_ = 0, transfer_calls_ = 0, op_calls_ = 0;

  std::vector<float> host_w_dx_; // only while the tile has no device
  float *w_ = nullptr;           // device [x][d]
  float *w_owned_ = nullptr;
  uint64_t shared_version_ = 0;
  float *delta_w_ = nullptr; // caller-owned target of the update in delta-weight mode
  float *w_fast_ = nullptr; // Transfer: fast (hidden) tile A, [x][d]
  float *t_buffer_ = nullptr; // buffered Transfer: digital buffer per element, [x][d]
  // dynamic Transfer: running mean of the reads and the reference mean per element, [x][d];
  // per line, whether its in chopper flipped at its previous transfer
  float *t_mean_ = nullptr, *t_past_ = nullptr;
  std::vector<unsigned char> chop_switched_;
  DeviceStore dev_[2];
  int n_dev_ = 1;
  // Transfer counters (rpu_transfer_device.cpp:396-516, rpu_vector_device.cpp:513-526)
  long long update_idx_ = 0;
  int slice_idx_ = 0;

  // scratch
  int scratch_m_ = 0;
  float *scale_ = nullptr, *factor_ = nullptr, *vnorm_ = nullptr, *sval_ = nullptr;
  int *flags_ = nullptr, *bm_stats_ = nullptr;
  // out_noise_std > 0: std-dev of the output noise of every output line, forward (d_size) and
  // backward (x_size), drawn once per tile (rpu_forward_backward_pass.cpp:306-313)
  float *f_onv_ = nullptr, *b_onv_ = nullptr;
  float *nm_state_ = nullptr;
  unsigned char *chop_in_ = nullptr, *chop_out_ = nullptr; // chopped transfer: x_size / d_size flags
  uint64_t chop_passes_ = 0;                               // full passes over the matrix (transfer_counter_)
  struct ChopRng { // host draws of the random in-chopper flips
    std::mt19937 gen{0x9e3779b9u};
    std::uniform_real_distribution<float> ud{0.0f, 1.0f};
    float uniform() { return ud(gen); }
  } chop_rng_;
  uint32_t *xls_ = nullptr, *xlx_ = nullptr, *xloff_ = nullptr; // compacted x lists (stream update)
  // per-line tables of a direction (MVParameter, rpu_forward_backward_pass.h:14-22)
  struct LineTables {
    std::vector<float> h_voff, h_nl, h_onv;
    float *voff = nullptr, *nl = nullptr;
    float nl_factor = 1.0f;
  };
  LineTables f_lt_, b_lt_;
  void populateLineTables();
  void uploadLineTables(LineTables &lt, const IOEff &io, int n, float **onv);
  void setLineTables(MvmProblem &p, const LineTables &lt, const float *onv) const;
  // power-law drift: per element the weight seen by the previous call, the weight and the time of
  // its last write, and (pulsed devices) its exponent; time in units of t0
  // modified copy of the weights that forward / backward read (modify_weights), its largest
  // magnitude (device scalar), and whether a test-mode forward reads it too
  float *fb_w_ = nullptr, *fb_amax_ = nullptr;
  bool fb_active_ = false, fb_in_test_ = false;
  uint64_t fb_version_ = 0;
  const float *fbWeights(bool is_test) const {
    return (fb_active_ && (!is_test || fb_in_test_)) ? fb_w_ : w_;
  }
  float *drift_prev_ = nullptr, *drift_w0_ = nullptr, *drift_t_ = nullptr, *drift_nu_ = nullptr;
  float drift_now_ = 0.0f;
  uint32_t *xw_ = nullptr, *dw_ = nullptr;
  // transposed x words [x_size][m_pad] and their bitmaps, for the streaming update of large batches
  uint32_t *xwt_ = nullptr, *xnzt_ = nullptr;
  size_t xwt_words_ = 0;
  void ensureStreamScratch(int m_pad);
  float *onehot_ = nullptr, *tread_ = nullptr;
  uint32_t *t_words_ = nullptr; // Tiki-Taka write: pulse words of its single sample
  // tensor-core engines (forward / backward operand caches), rebuilt when the weights change
  std::unique_ptr<TcEngine> tc_fwd_, tc_bwd_;
  uint64_t w_version_ = 1, tc_fwd_version_ = 0, tc_bwd_version_ = 0;
  // indexed interface: own copy of the index array, its largest entry, and the sample-major
  // matrices [n_img * m_batch][x_size] and [n_img * m_batch][d_size]
  int32_t *idx_ = nullptr;
  long long idx_cap_ = 0, idx_count_ = 0;
  int32_t idx_max_ = 0;
  float *cols_x_ = nullptr, *cols_d_ = nullptr;
  long long cols_x_cap_ = 0, cols_d_cap_ = 0;
  // the index array as [m_batch][x_size] for callers that hand it over as [x_size][m_batch]
  // (built on the first such call after set_matrix_indices)
  int32_t *idx_t_ = nullptr;
  long long idx_t_cap_ = 0;
  bool idx_t_valid_ = false;
  RowGather upd_gather_; // set around an update whose samples are gathered from images
  unsigned long long *pulses_up_ = nullptr, *pulses_down_ = nullptr; // count_pulses: [x][d] each
  // mixed-precision compound: digital accumulator chi ([x][d] like the weights), quantised
  // samples of the current batch, pulse counts / one-hot vectors of the rows in transfer, the
  // sample counter and the next row to transfer
  float *chi_ = nullptr, *mp_qx_ = nullptr, *mp_qd_ = nullptr, *mp_counts_ = nullptr, *mp_onehot_ = nullptr;
  int mp_q_cap_ = 0;
  long long mp_update_idx_ = 0;
  int mp_row_idx_ = 0;
  float mp_granularity_ = 0.0f;
  void updateMixed(UpdateProblem &u, cudaStream_t s);
  void transferMixed(cudaStream_t s);
  // inverse of the index array for the backward pass: for every image element the positions of
  // the index array that name it (CSR: csr_off_[e] .. csr_off_[e + 1] into csr_pos_), in
  // ascending order, so that the sum over them has a fixed order
  int32_t *csr_off_ = nullptr, *csr_pos_ = nullptr;
  long long csr_elems_ = 0; // image elements covered by the CSR (largest index - 1)
  unsigned char *clip_stats_ = nullptr; // statistics of clipWeights (sum, sum of squares, row maxima)
  // output block of a tile that adds to earlier in-splits under bound management
  float *acc_block_ = nullptr;
  size_t acc_block_floats_ = 0;
  // staging for the *_host entry points
  float *stage_dev_ = nullptr;
  float *stage_pinned_ = nullptr;
  size_t stage_floats_ = 0;
};

} // namespace ab200
