// extern "C" boundary of the library (declared in include/aihwkit_b200.h): translates C++
// exceptions into return codes + ab200_last_error(), like the reference's binding turns
// std::runtime_error into Python RuntimeError.
#include "array.h"
#include "tile.h"

#include <algorithm>
#include <mutex>
#include <cstdint>
#include <cstring>

namespace ab200 {
uint64_t launchCount();
}

using ab200::Tile;
using ab200::TileArray;

static thread_local std::string g_error;

namespace ab200 {
void setLastError(const char *msg) { g_error = msg ? msg : ""; }
} // namespace ab200

#define AB200_TRY try {
#define AB200_CATCH                                                                                \
  }                                                                                                \
  catch (const std::exception &e) {                                                                \
    g_error = e.what();                                                                            \
    return 1;                                                                                      \
  }                                                                                                \
  catch (...) {                                                                                    \
    g_error = "unknown error";                                                                     \
    return 1;                                                                                      \
  }                                                                                                \
  return 0;

// Every entry point holds the object's mutex for the duration of the call, as the reference's
// binding does (std::lock_guard on RPUSimple::mutex_, src/rpucuda/rpu.h:669,
// rpu_base_tiles.cpp:169,439,...): the handle is returned together with the lock.
template <class X> struct Locked {
  X *p;
  std::unique_lock<std::mutex> lock;
  X *operator->() const { return p; }
};
static Locked<Tile> T(ab200_tile *t) {
  if (!t) {
    AB200_FATAL("null tile handle");
  }
  Tile *x = reinterpret_cast<Tile *>(t);
  return Locked<Tile>{x, std::unique_lock<std::mutex>(x->mutex())};
}
static Locked<const Tile> T(const ab200_tile *t) {
  if (!t) {
    AB200_FATAL("null tile handle");
  }
  const Tile *x = reinterpret_cast<const Tile *>(t);
  return Locked<const Tile>{x, std::unique_lock<std::mutex>(x->mutex())};
}
static Locked<TileArray> A(ab200_array *a) {
  if (!a) {
    AB200_FATAL("null array handle");
  }
  TileArray *x = reinterpret_cast<TileArray *>(a);
  return Locked<TileArray>{x, std::unique_lock<std::mutex>(x->mutex())};
}

extern "C" {

const char *ab200_last_error(void) { return g_error.c_str(); }
const char *ab200_version(void) { return "aihwkit_b200 0.1.0 (sm_100a)"; }
size_t ab200_sizeof(int which) {
  switch (which) {
  case 0: return sizeof(ab200_io_params);
  case 1: return sizeof(ab200_update_params);
  case 2: return sizeof(ab200_device_params);
  case 3: return sizeof(ab200_transfer_params);
  case 4: return sizeof(ab200_tile_config);
  case 5: return sizeof(ab200_scatter_plan);
  case 6: return sizeof(ab200_mixedprec_params);
  default: return 0;
  }
}

void ab200_default_io_params(ab200_io_params *io) {
  std::memset(io, 0, sizeof(*io));
  io->noise_management = AB200_NM_ABS_MAX;
  io->bound_management = AB200_BM_NONE;
  io->w_noise_type = AB200_WNOISE_NONE;
  io->bm_test_negative_bound = 1;
  io->max_bm_factor = 1000;
  io->inp_bound = 1.0f;
  io->inp_res = 1.0f / 126.0f;
  io->out_bound = 12.0f;
  io->out_res = 1.0f / 510.0f;
  io->nm_assumed_wmax = 0.6f;
  io->out_noise = 0.06f;
  io->out_scale = 1.0f;
  io->nm_decay = 1e-3f;
  io->ir_drop_g_ratio = 5.7143e5f;
  io->slope_calibration = 0.5f;
  io->mv_type = AB200_MV_ONE_PASS;
  io->max_bm_res = 0.25f;
}

void ab200_default_update_params(ab200_update_params *up) {
  std::memset(up, 0, sizeof(*up));
  up->pulse_type = AB200_PULSE_STOCHASTIC_COMPRESSED;
  up->desired_bl = 31;
  up->fixed_bl = 1;
  up->update_management = 1;
  up->update_bl_management = 1;
  up->um_grad_scale = 1.0f;
}

void ab200_default_device_params(ab200_device_params *dp, int32_t kind) {
  std::memset(dp, 0, sizeof(*dp));
  dp->kind = kind;
  dp->dw_min = 0.001f;
  dp->dw_min_dtod = 0.3f;
  dp->dw_min_std = 0.3f;
  dp->w_min = -0.6f;
  dp->w_min_dtod = 0.3f;
  dp->w_max = 0.6f;
  dp->w_max_dtod = 0.3f;
  dp->up_down_dtod = 0.01f;
  dp->ls_mult_noise = 1;
  dp->ls_mean_bound_reference = 1;
  dp->ls_decrease_up_dtod = 0.05f;
  dp->ls_decrease_down_dtod = 0.05f;
  dp->es_A_up = 0.00081f;
  dp->es_A_down = 0.36833f;
  dp->es_gamma_up = 12.44625f;
  dp->es_gamma_down = 12.78785f;
  dp->es_a = 0.244f;
  dp->es_b = 0.2425f;
  dp->ps_gamma = 1.0f; /* rpu_powstep_device.h:22-25 */
  dp->ps_gamma_dtod = 0.1f;
  dp->ps_gamma_up_down = 0.0f;
  dp->ps_gamma_up_down_dtod = 0.0f;
  dp->pw_n = 1; /* rpu_piecewisestep_device.h:24-25 */
  dp->pw_up[0] = dp->pw_down[0] = 1.0f;
  dp->drift.wg_ratio = 1.0f; /* weight_drifter.h:17-45 */
  dp->drift.t0 = 1.0f;
  dp->drift.reset_tol = 1e-7f;
  if (kind == AB200_DEVICE_SOFT_BOUNDS) {
    dp->ls_decrease_up = dp->ls_decrease_down = 1.0f;
    dp->ls_decrease_up_dtod = dp->ls_decrease_down_dtod = 0.0f;
    dp->ls_mean_bound_reference = 0;
  }
}

void ab200_default_transfer_params(ab200_transfer_params *tp) {
  std::memset(tp, 0, sizeof(*tp));
  tp->transfer_every = 1.0f;
  tp->n_reads_per_transfer = 1;
  tp->in_chop_prob = 1.0f; /* rpu_chopped_transfer_device.h:24-37 */
  tp->in_chop_random = 1;
  tp->buffer_granularity = 1.0f;
  tp->tail_weightening = 1.0f; /* rpu_dynamic_transfer_device.h:28-29 */
  tp->buffer_cap = 10.0f;
  tp->thres_scale = 1.0f;
  tp->step = 1.0f;
  tp->forget_buffer = 1;
  tp->transfer_lr = 1.0f;
  tp->scale_transfer_lr = 1;
  tp->scale_fast_lr = 1;
  tp->transfer_columns = 1;
  ab200_default_io_params(&tp->transfer_io);
  ab200_default_update_params(&tp->transfer_up);
}

void ab200_default_mixedprec_params(ab200_mixedprec_params *mp) {
  std::memset(mp, 0, sizeof(*mp));
  mp->transfer_every = 1; /* rpu_mixedprec_device_base.h:26-31, rpu_mixedprec_device.h:32-36 */
  mp->n_rows_per_transfer = -1;
  mp->transfer_lr = 1.0f;
}

int ab200_tile_create(const ab200_tile_config *cfg, int cuda_device, ab200_tile **out) {
  AB200_TRY
  if (!cfg || !out) {
    AB200_FATAL("null argument");
  }
  *out = reinterpret_cast<ab200_tile *>(new Tile(*cfg, cuda_device));
  AB200_CATCH
}

int ab200_tile_destroy(ab200_tile *tile) {
  AB200_TRY
  delete reinterpret_cast<Tile *>(tile);
  AB200_CATCH
}

int ab200_tile_to_device(ab200_tile *tile, int cuda_device) {
  AB200_TRY
  T(tile)->toDevice(cuda_device);
  AB200_CATCH
}

int ab200_tile_get_x_size(const ab200_tile *tile) { return tile ? T(tile)->xSize() : -1; }
int ab200_tile_get_d_size(const ab200_tile *tile) { return tile ? T(tile)->dSize() : -1; }

int ab200_tile_set_learning_rate(ab200_tile *tile, float lr) {
  AB200_TRY
  T(tile)->setLearningRate(lr);
  AB200_CATCH
}
int ab200_tile_get_learning_rate(const ab200_tile *tile, float *lr) {
  AB200_TRY
  *lr = T(tile)->learningRate();
  AB200_CATCH
}

int ab200_tile_set_weights(ab200_tile *tile, const float *w_host) {
  AB200_TRY
  T(tile)->setWeights(w_host);
  AB200_CATCH
}
int ab200_tile_get_weights(ab200_tile *tile, float *w_host) {
  AB200_TRY
  T(tile)->getWeights(w_host);
  AB200_CATCH
}
int ab200_tile_set_weights_device(ab200_tile *tile, const float *w_dev_xd, void *stream) {
  AB200_TRY
  if (!w_dev_xd) {
    AB200_FATAL("null weight pointer");
  }
  T(tile)->setWeightsDevice(w_dev_xd, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_get_weights_device(ab200_tile *tile, float *w_dev_xd, void *stream) {
  AB200_TRY
  T(tile)->getWeightsDevice(w_dev_xd, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_set_shared_weights(ab200_tile *tile, float *w_dev_xd, uint64_t version) {
  AB200_TRY
  T(tile)->setSharedWeights(w_dev_xd, version);
  AB200_CATCH
}

int ab200_tile_set_delta_weights(ab200_tile *tile, float *dw_dev_xd) {
  AB200_TRY
  T(tile)->setDeltaWeights(dw_dev_xd);
  AB200_CATCH
}

int ab200_tile_hidden_parameter_count(const ab200_tile *tile) {
  return tile ? T(tile)->hiddenCount() : 0;
}
const char *ab200_tile_hidden_parameter_name(const ab200_tile *tile, int index) {
  return tile ? T(tile)->hiddenName(index) : "";
}
int ab200_tile_get_hidden_parameters(ab200_tile *tile, float *out_host) {
  AB200_TRY
  T(tile)->getHidden(out_host);
  AB200_CATCH
}
int ab200_tile_set_hidden_parameters(ab200_tile *tile, const float *in_host) {
  AB200_TRY
  T(tile)->setHidden(in_host);
  AB200_CATCH
}

static void checkBatch(int m) {
  if (m < 0) {
    AB200_FATAL("m_batch must be >= 0");
  }
}

int ab200_tile_forward(ab200_tile *tile, const float *x_dev, float *d_dev, int bias, int m_batch,
                       int x_trans, int d_trans, int is_test, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->forward(x_dev, d_dev, bias != 0, m_batch, x_trans != 0, d_trans != 0, is_test != 0,
                   (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_backward(ab200_tile *tile, const float *d_dev, float *x_dev, int bias, int m_batch,
                        int d_trans, int x_trans, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->backward(d_dev, x_dev, bias != 0, m_batch, d_trans != 0, x_trans != 0,
                    (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_update(ab200_tile *tile, const float *x_dev, const float *d_dev, int bias,
                      int m_batch, int x_trans, int d_trans, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->update(x_dev, d_dev, bias != 0, m_batch, x_trans != 0, d_trans != 0,
                  (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_forward_host(ab200_tile *tile, const float *x_host, float *d_host, int bias,
                            int m_batch, int x_trans, int d_trans, int is_test, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->forwardHost(x_host, d_host, bias != 0, m_batch, x_trans != 0, d_trans != 0,
                       is_test != 0, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_backward_host(ab200_tile *tile, const float *d_host, float *x_host, int bias,
                             int m_batch, int d_trans, int x_trans, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->backwardHost(d_host, x_host, bias != 0, m_batch, d_trans != 0, x_trans != 0,
                        (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_tile_update_host(ab200_tile *tile, const float *x_host, const float *d_host, int bias,
                           int m_batch, int x_trans, int d_trans, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  T(tile)->updateHost(x_host, d_host, bias != 0, m_batch, x_trans != 0, d_trans != 0,
                      (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_coincidences(ab200_tile *tile, const float *x_dev, const float *d_dev,
                            int32_t *counts_dev, void *stream) {
  AB200_TRY
  T(tile)->coincidences(x_dev, d_dev, counts_dev, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_set_matrix_indices(ab200_tile *tile, const int32_t *indices, long long count,
                                  void *stream) {
  AB200_TRY
  T(tile)->setMatrixIndices(indices, count, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_has_matrix_indices(ab200_tile *tile) {
  return tile != nullptr && T(tile)->hasMatrixIndices() ? 1 : 0;
}

int ab200_tile_forward_indexed(ab200_tile *tile, const float *x_dev, float *d_dev,
                               long long total_input_size, int m_batch, int dim3, int trans,
                               int is_test, void *stream) {
  AB200_TRY
  T(tile)->forwardIndexed(x_dev, d_dev, total_input_size, m_batch, dim3, trans != 0, is_test != 0,
                          (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_backward_indexed(ab200_tile *tile, const float *d_dev, float *x_dev,
                                long long total_output_size, int m_batch, int dim3, int trans,
                                void *stream) {
  AB200_TRY
  T(tile)->backwardIndexed(d_dev, x_dev, total_output_size, m_batch, dim3, trans != 0,
                           (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_update_indexed(ab200_tile *tile, const float *x_dev, const float *d_dev,
                              long long total_input_size, int m_batch, int dim3, int trans,
                              void *stream) {
  AB200_TRY
  T(tile)->updateIndexed(x_dev, d_dev, total_input_size, m_batch, dim3, trans != 0,
                         (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_extra_count(void) { return ab200::Tile::extraCount(); }

const char *ab200_tile_extra_name(int k) {
  try {
    return ab200::Tile::extraName(k);
  } catch (const std::exception &e) {
    g_error = e.what();
    return nullptr;
  }
}

int ab200_tile_dump_extra(ab200_tile *tile, double *values) {
  AB200_TRY
  T(tile)->dumpExtra(values);
  AB200_CATCH
}

int ab200_tile_load_extra(ab200_tile *tile, const char *const *names, const double *values,
                          int count, int strict) {
  AB200_TRY
  T(tile)->loadExtra(names, values, count, strict != 0);
  AB200_CATCH
}

int ab200_tile_get_io_vector(ab200_tile *tile, int backward, int which, float *values_host, int n) {
  AB200_TRY
  T(tile)->getIoVector(backward != 0, which, values_host, n);
  AB200_CATCH
}

int ab200_tile_set_io_vector(ab200_tile *tile, int backward, int which, const float *values_host,
                             int n) {
  AB200_TRY
  T(tile)->setIoVector(backward != 0, which, values_host, n);
  AB200_CATCH
}

int ab200_tile_modify_weights(ab200_tile *tile, const ab200_weight_modifier_params *params,
                              void *stream) {
  AB200_TRY
  if (!params) {
    AB200_FATAL("modify_weights: null parameters");
  }
  T(tile)->modifyWeights(*params, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_drift_weights(ab200_tile *tile, float time_since_last_call, void *stream) {
  AB200_TRY
  T(tile)->driftWeights(time_since_last_call, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_decay_weights(ab200_tile *tile, float alpha, int bias_no_decay, void *stream) {
  AB200_TRY
  T(tile)->decayWeights(alpha, bias_no_decay != 0, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_diffuse_weights(ab200_tile *tile, void *stream) {
  AB200_TRY
  T(tile)->diffuseWeights((cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_clip_weights(ab200_tile *tile, int clip_type, float fixed_value, float sigma,
                            void *stream) {
  AB200_TRY
  T(tile)->clipWeights(clip_type, fixed_value, sigma, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_reset_columns(ab200_tile *tile, int start_col, int n_cols, float reset_prob,
                             void *stream) {
  AB200_TRY
  T(tile)->resetColumns(start_col, n_cols, reset_prob, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_set_weights_uniform_random(ab200_tile *tile, float min_value, float max_value,
                                          void *stream) {
  AB200_TRY
  T(tile)->setWeightsUniformRandom(min_value, max_value, (cudaStream_t)stream);
  AB200_CATCH
}

int ab200_tile_extra_vector_count(const ab200_tile *tile) {
  try {
    return tile ? T(tile)->extraVectorCount() : 0;
  } catch (...) {
    return 0;
  }
}
const char *ab200_tile_extra_vector_name(const ab200_tile *tile, int k) {
  try {
    return T(tile)->extraVectorName(k);
  } catch (...) {
    return "";
  }
}
int ab200_tile_extra_vector_size(const ab200_tile *tile, int k) {
  try {
    return T(tile)->extraVectorSize(k);
  } catch (...) {
    return 0;
  }
}
int ab200_tile_get_extra_vector(ab200_tile *tile, int k, double *out) {
  AB200_TRY
  if (!out) {
    AB200_FATAL("null argument");
  }
  T(tile)->getExtraVector(k, out);
  AB200_CATCH
}
int ab200_tile_set_extra_vector(ab200_tile *tile, int k, const double *in, int n) {
  AB200_TRY
  if (!in) {
    AB200_FATAL("null argument");
  }
  T(tile)->setExtraVector(k, in, n);
  AB200_CATCH
}

int ab200_tile_get_pulse_counters(ab200_tile *tile, int64_t *out_host) {
  AB200_TRY
  if (!out_host) {
    AB200_FATAL("null argument");
  }
  T(tile)->getPulseCounters(out_host);
  AB200_CATCH
}

int ab200_tile_counts_pulses(ab200_tile *tile) {
  try {
    return tile && T(tile)->countsPulses() ? 1 : 0;
  } catch (...) {
    return 0;
  }
}

int ab200_tile_last_bm_stats(ab200_tile *tile, int32_t *n_rerun_samples, float *max_reduction) {
  AB200_TRY
  T(tile)->lastBmStats(n_rerun_samples, max_reduction);
  AB200_CATCH
}

int ab200_tile_set_seed(ab200_tile *tile, uint64_t seed) {
  AB200_TRY
  T(tile)->setSeed(seed);
  AB200_CATCH
}

int ab200_array_create(const ab200_tile_config *cfg, int out_size, int in_size,
                       int max_output_size, int max_input_size, int in_split_begin,
                       int in_split_end, int cuda_device, ab200_array **out) {
  AB200_TRY
  if (!cfg || !out) {
    AB200_FATAL("null argument");
  }
  if (cuda_device < 0) {
    AB200_FATAL("the mapped-tile array needs a CUDA device");
  }
  *out = reinterpret_cast<ab200_array *>(new TileArray(*cfg, out_size, in_size, max_output_size,
                                                       max_input_size, in_split_begin,
                                                       in_split_end, cuda_device));
  AB200_CATCH
}
int ab200_array_create_block(const ab200_tile_config *cfg, int out_size, int in_size,
                             int max_output_size, int max_input_size, int in_split_begin,
                             int in_split_end, int out_split_begin, int out_split_end,
                             int cuda_device, ab200_array **out) {
  AB200_TRY
  if (!cfg || !out) {
    AB200_FATAL("null argument");
  }
  if (cuda_device < 0) {
    AB200_FATAL("the mapped-tile array needs a CUDA device");
  }
  *out = reinterpret_cast<ab200_array *>(new TileArray(*cfg, out_size, in_size, max_output_size,
                                                       max_input_size, in_split_begin, in_split_end,
                                                       cuda_device, out_split_begin, out_split_end));
  AB200_CATCH
}

int ab200_array_destroy(ab200_array *arr) {
  AB200_TRY
  delete reinterpret_cast<TileArray *>(arr);
  AB200_CATCH
}
int ab200_array_num_in_splits(const ab200_array *arr) {
  return arr ? reinterpret_cast<const TileArray *>(arr)->numInSplits() : -1;
}
int ab200_array_num_out_splits(const ab200_array *arr) {
  return arr ? reinterpret_cast<const TileArray *>(arr)->numOutSplits() : -1;
}
int ab200_array_set_weights(ab200_array *arr, const float *w_host) {
  AB200_TRY
  A(arr)->setWeights(w_host);
  AB200_CATCH
}
int ab200_array_backward(ab200_array *arr, const float *d_dev, float *x_grad_dev, int m_batch,
                         void *stream) {
  AB200_TRY
  A(arr)->backward(d_dev, x_grad_dev, m_batch, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_array_update(ab200_array *arr, const float *x_dev, const float *d_dev, int m_batch,
                       void *stream) {
  AB200_TRY
  A(arr)->update(x_dev, d_dev, m_batch, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_array_set_learning_rate(ab200_array *arr, float lr) {
  AB200_TRY
  A(arr)->setLearningRate(lr);
  AB200_CATCH
}
int ab200_array_forward_scatter(ab200_array *arr, const float *x_local_dev, int m_batch,
                                float *const *out_table_dev, int n_owners, int rows_per_owner,
                                int rotate_rows, void *stream) {
  AB200_TRY
  A(arr)->forwardScatter(x_local_dev, m_batch, out_table_dev, n_owners, rows_per_owner, rotate_rows,
                         (cudaStream_t)stream);
  AB200_CATCH
}

namespace {
// Count of waits that ran out, in page-locked host memory the kernels write through a mapped
// pointer: one word per device, created on first use.
constexpr int kMaxWaitDevices = 64;
int *g_wait_host[kMaxWaitDevices] = {nullptr};
int *g_wait_dev[kMaxWaitDevices] = {nullptr};
std::mutex g_wait_mu;

int *waitStatusWord(int dev) {
  if (dev < 0 || dev >= kMaxWaitDevices) {
    AB200_FATAL("unsupported device index " << dev);
  }
  std::lock_guard<std::mutex> lock(g_wait_mu);
  if (!g_wait_host[dev]) {
    AB200_CUDA(cudaHostAlloc(&g_wait_host[dev], sizeof(int), cudaHostAllocMapped));
    *g_wait_host[dev] = 0;
    AB200_CUDA(cudaHostGetDevicePointer(&g_wait_dev[dev], g_wait_host[dev], 0));
  }
  return g_wait_dev[dev];
}

// Thread 0 of every CTA waits (bounded) until all flags have reached `epoch`; false = gave up.
__device__ __forceinline__ bool waitFlags(const int *flags, int n_flags, int epoch,
                                          long long max_cycles, int *status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (int k = 0; k < n_flags && ok; k++) {
      unsigned pause = 32;
      while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + k) : "memory");
        if (v - epoch >= 0) {
          break;
        }
        if (clock64() - t0 > max_cycles) {
          ok = 0;
          break;
        }
        __nanosleep(pause);
        pause = pause < 1024u ? pause * 2u : pause;
      }
    }
    if (!ok && blockIdx.x == 0) {
      atomicAdd_system(status, 1);
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

long long waitCycles(float max_wait_ms, int dev) {
  // the clock-rate attribute is a slow driver query (about a millisecond): once per device
  static int khz_of[kMaxWaitDevices] = {0};
  int khz = dev >= 0 && dev < kMaxWaitDevices ? khz_of[dev] : 0;
  if (khz == 0) {
    AB200_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    if (dev >= 0 && dev < kMaxWaitDevices) {
      khz_of[dev] = khz;
    }
  }
  if (!(max_wait_ms > 0.0f)) {
    max_wait_ms = 2000.0f;
  }
  return (long long)((double)max_wait_ms * (double)(khz > 0 ? khz : 1500000));
}
} // namespace

namespace {
__global__ void __launch_bounds__(256)
    sumSlotsKernel(const float4 *slots, int n_slots, long long elems4, float4 *out) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= elems4) {
    return;
  }
  float4 acc = slots[t];
  for (int k = 1; k < n_slots; k++) {
    const float4 v = slots[(long long)k * elems4 + t];
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  out[t] = acc;
}
} // namespace

int ab200_sum_slots(const float *slots_dev, int n_slots, long long elems, float *out_dev,
                    void *stream) {
  AB200_TRY
  if (n_slots <= 0 || elems <= 0) {
    AB200_FATAL("sum_slots: nothing to add");
  }
  if ((elems & 3) != 0 || (((uintptr_t)slots_dev | (uintptr_t)out_dev) & 15) != 0) {
    AB200_FATAL("sum_slots: element count must be a multiple of 4 and the buffers 16-byte aligned");
  }
  const long long e4 = elems / 4;
  sumSlotsKernel<<<(unsigned)((e4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const float4 *)slots_dev, n_slots, e4, (float4 *)out_dev);
  AB200_LAUNCH_CHECK();
  AB200_CATCH
}

int ab200_array_scatter_codes_supported(ab200_array *arr) {
  try {
    auto a = A(arr);
    return a->scatterCodesSupported() ? 1 : 0;
  } catch (...) {
    return 0;
  }
}
int ab200_array_forward_scatter_codes(ab200_array *arr, const float *x_local_dev, int m_batch,
                                      unsigned char *const *code_table_dev,
                                      float *const *fac_table_dev, int n_owners,
                                      int rows_per_owner, int rotate_rows, void *stream) {
  AB200_TRY
  A(arr)->forwardScatterCodes(x_local_dev, m_batch, code_table_dev, fac_table_dev, n_owners,
                              rows_per_owner, rotate_rows, (cudaStream_t)stream);
  AB200_CATCH
}

namespace {
struct CodeSlots {
  const unsigned char *codes;
  long long code_stride;
  const float *facs;
  long long fac_stride;
  int n_slots;
  int n_planes[16];
  int rows_per_owner, rows_valid, out_size;
  float *out;
  // optional: rows [row0, rows_valid) only, after the flags have reached `epoch`
  int row0;
  const int *flags;
  int n_flags, epoch;
  long long max_cycles;
  int *status;
};

// one thread per row and four columns: the word of four codes of every slot and plane, times the
// row's factor; planes of a slot first (fused multiply-add chain from zero, as the MVM kernel sums
// its in-splits), then the slots in order (as sumSlotsKernel adds them)
__global__ void __launch_bounds__(256) codeSlotsKernel(CodeSlots p) {
  ab200::pdlEnter(); // launched behind the scatter kernel of the same step: no launch gap between them
  if (p.n_flags > 0 && !waitFlags(p.flags, p.n_flags, p.epoch, p.max_cycles, p.status)) {
    return;
  }
  const int w4 = p.out_size >> 2;
  const long long t = (long long)p.row0 * w4 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= (long long)p.rows_valid * w4) {
    return;
  }
  const int row = (int)(t / w4), c4 = (int)(t % w4);
  const int col = c4 * 4;
  const long long plane_bytes = (long long)p.rows_per_owner * p.out_size;
  const long long off = ((long long)(row >> 5) * (p.out_size >> 5) + (col >> 5)) * 1024 +
                        (long long)(row & 31) * 32 + (col & 31);
  float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int q = 0; q < p.n_slots; q++) {
    const unsigned char *cs = p.codes + (long long)q * p.code_stride;
    const float *fs = p.facs + (long long)q * p.fac_stride;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < p.n_planes[q]; i++) {
      const uint32_t w = *reinterpret_cast<const uint32_t *>(cs + (long long)i * plane_bytes + off);
      const float f = fs[(long long)i * p.rows_per_owner + row];
      acc.x = fmaf((float)(signed char)(w & 0xFF), f, acc.x);
      acc.y = fmaf((float)(signed char)((w >> 8) & 0xFF), f, acc.y);
      acc.z = fmaf((float)(signed char)((w >> 16) & 0xFF), f, acc.z);
      acc.w = fmaf((float)(signed char)(w >> 24), f, acc.w);
    }
    if (q == 0) {
      total = acc;
    } else {
      total.x += acc.x;
      total.y += acc.y;
      total.z += acc.z;
      total.w += acc.w;
    }
  }
  *reinterpret_cast<float4 *>(p.out + (long long)row * p.out_size + col) = total;
}
} // namespace

int ab200_sum_code_slots(const unsigned char *code_slots_dev, long long code_slot_stride,
                         const float *fac_slots_dev, long long fac_slot_stride, int n_slots,
                         const int *n_planes, int rows_per_owner, int rows_valid, int out_size,
                         float *out_dev, void *stream) {
  AB200_TRY
  if (n_slots <= 0 || n_slots > 16 || n_planes == nullptr || rows_valid < 0 ||
      rows_valid > rows_per_owner || (rows_per_owner & 31) != 0 || (out_size & 31) != 0 ||
      (((uintptr_t)out_dev) & 15) != 0 || (((uintptr_t)code_slots_dev | (uintptr_t)code_slot_stride) & 3) != 0) {
    AB200_FATAL("sum_code_slots: 1..16 slots, rows and columns in multiples of 32, aligned buffers");
  }
  if (rows_valid == 0) {
    return 0;
  }
  CodeSlots p{};
  p.codes = code_slots_dev;
  p.code_stride = code_slot_stride;
  p.facs = fac_slots_dev;
  p.fac_stride = fac_slot_stride;
  p.n_slots = n_slots;
  for (int q = 0; q < n_slots; q++) {
    p.n_planes[q] = n_planes[q];
  }
  p.rows_per_owner = rows_per_owner;
  p.rows_valid = rows_valid;
  p.out_size = out_size;
  p.out = out_dev;
  const long long n = (long long)rows_valid * (out_size >> 2);
  AB200_CUDA(ab200::launchChained(codeSlotsKernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                  (cudaStream_t)stream, p));
  AB200_LAUNCH_CHECK();
  AB200_CATCH
}

int ab200_sum_code_slots_wait(const unsigned char *code_slots_dev, long long code_slot_stride,
                              const float *fac_slots_dev, long long fac_slot_stride, int n_slots,
                              const int *n_planes, int rows_per_owner, int row0, int rows,
                              int out_size, float *out_dev, const int32_t *flags_dev, int n_flags,
                              int epoch, float max_wait_ms, void *stream) {
  AB200_TRY
  if (n_slots <= 0 || n_slots > 16 || n_planes == nullptr || rows < 0 || row0 < 0 ||
      row0 + rows > rows_per_owner || (rows_per_owner & 31) != 0 || (out_size & 31) != 0 ||
      (((uintptr_t)out_dev) & 15) != 0 || (((uintptr_t)code_slots_dev | (uintptr_t)code_slot_stride) & 3) != 0) {
    AB200_FATAL("sum_code_slots_wait: 1..16 slots, rows and columns in multiples of 32, aligned buffers");
  }
  if (rows == 0) {
    return 0;
  }
  int dev = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  CodeSlots p{};
  p.codes = code_slots_dev;
  p.code_stride = code_slot_stride;
  p.facs = fac_slots_dev;
  p.fac_stride = fac_slot_stride;
  p.n_slots = n_slots;
  for (int q = 0; q < n_slots; q++) {
    p.n_planes[q] = n_planes[q];
  }
  p.rows_per_owner = rows_per_owner;
  p.row0 = row0;
  p.rows_valid = row0 + rows;
  p.out_size = out_size;
  p.out = out_dev;
  p.flags = flags_dev;
  p.n_flags = flags_dev ? n_flags : 0;
  p.epoch = epoch;
  p.max_cycles = waitCycles(max_wait_ms, dev);
  p.status = waitStatusWord(dev);
  const long long n = (long long)rows * (out_size >> 2);
  codeSlotsKernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p);
  AB200_LAUNCH_CHECK();
  AB200_CATCH
}

int ab200_array_forward_scatter_plan(ab200_array *arr, const float *x_local_dev, int m_batch,
                                     const ab200_scatter_plan *plan, void *stream) {
  AB200_TRY
  if (!plan) {
    AB200_FATAL("forward_scatter: null plan");
  }
  A(arr)->forwardScatterPlan(x_local_dev, m_batch, *plan, (cudaStream_t)stream);
  AB200_CATCH
}

namespace {
__global__ void __launch_bounds__(256)
    sumSlotsWaitKernel(const float4 *slots, int n_slots, long long stride4, long long e0, long long e1,
                       float4 *out, const int *flags, int n_flags, int epoch, long long max_cycles,
                       int *status) {
  ab200::pdlEnter();
  if (n_flags > 0 && !waitFlags(flags, n_flags, epoch, max_cycles, status)) {
    return;
  }
  const long long t = e0 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t >= e1) {
    return;
  }
  float4 acc = slots[t];
  for (int k = 1; k < n_slots; k++) {
    const float4 v = slots[(long long)k * stride4 + t];
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  out[t] = acc;
}

} // namespace

int ab200_sum_slots_wait(const float *slots_dev, int n_slots, long long slot_stride, int row0,
                         int rows, int out_size, float *out_dev, const int32_t *flags_dev,
                         int n_flags, int epoch, float max_wait_ms, void *stream) {
  AB200_TRY
  if (n_slots <= 0 || rows < 0 || row0 < 0 || out_size <= 0) {
    AB200_FATAL("sum_slots_wait: invalid sizes");
  }
  if ((out_size & 3) != 0 || (slot_stride & 3) != 0 ||
      (((uintptr_t)slots_dev | (uintptr_t)out_dev) & 15) != 0) {
    AB200_FATAL("sum_slots_wait: sizes must be multiples of 4 floats and the buffers 16-byte aligned");
  }
  if (rows == 0) {
    return 0;
  }
  int dev = 0;
  AB200_CUDA(cudaGetDevice(&dev));
  int *status = waitStatusWord(dev);
  const long long e0 = (long long)row0 * out_size / 4, e1 = (long long)(row0 + rows) * out_size / 4;
  AB200_CUDA(ab200::launchChained(sumSlotsWaitKernel, dim3((unsigned)((e1 - e0 + 255) / 256)), dim3(256), 0,
                                  (cudaStream_t)stream, (const float4 *)slots_dev, n_slots, slot_stride / 4,
                                  e0, e1, (float4 *)out_dev, flags_dev, flags_dev ? n_flags : 0, epoch,
                                  waitCycles(max_wait_ms, dev), status));
  AB200_LAUNCH_CHECK();
  AB200_CATCH
}

int ab200_measure_popc_peak(int cuda_device, double *pairs_per_s) {
  AB200_TRY
  if (!pairs_per_s) {
    AB200_FATAL("measure_popc_peak: null pointer");
  }
  AB200_CUDA(cudaSetDevice(cuda_device));
  *pairs_per_s = ab200::measurePopcPeak(nullptr);
  AB200_CATCH
}

int ab200_wait_status(int cuda_device, int *timed_out) {
  AB200_TRY
  if (!timed_out) {
    AB200_FATAL("wait_status: null pointer");
  }
  *timed_out = 0;
  if (cuda_device >= 0 && cuda_device < kMaxWaitDevices) {
    std::lock_guard<std::mutex> lock(g_wait_mu);
    if (g_wait_host[cuda_device]) {
      *timed_out = *(volatile int *)g_wait_host[cuda_device];
      *(volatile int *)g_wait_host[cuda_device] = 0;
    }
  }
  AB200_CATCH
}

int ab200_peer_alloc(size_t bytes, int cuda_device, void **dev_ptr, unsigned char handle_out[64]) {
  AB200_TRY
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  AB200_CUDA(cudaSetDevice(cuda_device));
  void *p = nullptr;
  AB200_CUDA(cudaMalloc(&p, bytes));
  // slots of ranks that never write (they own no in-split) and rows beyond the batch are summed
  // like any others: they must read as zero
  cudaError_t ez = cudaMemset(p, 0, bytes);
  if (ez != cudaSuccess) {
    cudaFree(p);
    AB200_FATAL("cudaMemset of the peer buffer failed: " << cudaGetErrorString(ez));
  }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    AB200_FATAL("cudaIpcGetMemHandle failed: " << cudaGetErrorString(e));
  }
  std::memcpy(handle_out, &h, 64);
  *dev_ptr = p;
  AB200_CATCH
}

int ab200_peer_open(const unsigned char handle[64], int cuda_device, void **dev_ptr) {
  AB200_TRY
  AB200_CUDA(cudaSetDevice(cuda_device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void *p = nullptr;
  AB200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *dev_ptr = p;
  AB200_CATCH
}

int ab200_peer_close(void *dev_ptr) {
  AB200_TRY
  AB200_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  AB200_CATCH
}

int ab200_peer_free(void *dev_ptr) {
  AB200_TRY
  AB200_CUDA(cudaFree(dev_ptr));
  AB200_CATCH
}

int ab200_array_set_weights_scaled(ab200_array *arr, const float *w_host, float omega) {
  AB200_TRY
  A(arr)->setWeights(w_host, omega);
  AB200_CATCH
}
int ab200_array_get_tile_scales(ab200_array *arr, float *scales_host) {
  AB200_TRY
  const std::vector<float> &sc = A(arr)->tileScales();
  std::copy(sc.begin(), sc.end(), scales_host);
  AB200_CATCH
}
int ab200_array_set_bias(ab200_array *arr, const float *bias_host) {
  AB200_TRY
  A(arr)->setBias(bias_host);
  AB200_CATCH
}
int ab200_array_get_weights(ab200_array *arr, float *w_host) {
  AB200_TRY
  A(arr)->getWeights(w_host);
  AB200_CATCH
}
int ab200_array_forward(ab200_array *arr, const float *x_dev, float *y_dev, int m_batch,
                        int is_test, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  A(arr)->forward(x_dev, y_dev, m_batch, is_test != 0, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_array_forward_local(ab200_array *arr, const float *x_local_dev, float *y_dev,
                              int m_batch, int is_test, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  A(arr)->forwardLocal(x_local_dev, y_dev, m_batch, is_test != 0, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_array_local_in_size(const ab200_array *arr) {
  return arr ? reinterpret_cast<const TileArray *>(arr)->localInSize() : -1;
}
int ab200_array_forward_host(ab200_array *arr, const float *x_host, float *y_host, int m_batch,
                             int is_test, void *stream) {
  AB200_TRY
  checkBatch(m_batch);
  A(arr)->forwardHost(x_host, y_host, m_batch, is_test != 0, (cudaStream_t)stream);
  AB200_CATCH
}
int ab200_array_set_seed(ab200_array *arr, uint64_t seed) {
  AB200_TRY
  A(arr)->setSeed(seed);
  AB200_CATCH
}

int ab200_set_mvm_path(int mode) {
  AB200_TRY
  if (mode < 0 || mode > 3) {
    AB200_FATAL("mvm path mode must be 0, 1, 2 or 3");
  }
  ab200::setMvmPath(mode);
  AB200_CATCH
}

int ab200_set_update_path(int mode) {
  AB200_TRY
  if (mode < 0 || mode > 2) {
    AB200_FATAL("set_update_path: mode must be 0, 1 or 2");
  }
  ab200::setUpdatePath(mode);
  AB200_CATCH
}

uint64_t ab200_kernel_launch_count(void) { return ab200::launchCount(); }

} // extern "C"
