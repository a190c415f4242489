// Mapped-tile layer: a logical [out_size][in_size] weight split into physical tiles
// (TileModuleArray, src/aihwkit/simulator/tiles/array.py:30-198).
#pragma once

#include "tc_engine.h"
#include "tile.h"

#include <memory>
#include <mutex>
#include <vector>

namespace ab200 {

std::vector<int> splitSizes(int size, int split_max);

class TileArray {
public:
  // [in_begin, in_end) x [out_begin, out_end): the in-splits and out-splits this object
  // materialises (a shard of the layer); an end of -1 means "to the last one"
  TileArray(const ab200_tile_config &cfg, int out_size, int in_size, int max_out, int max_in,
            int in_begin, int in_end, int cuda_device, int out_begin = 0, int out_end = -1);
  ~TileArray();
  std::mutex &mutex() const { return mu_; }
  int numInSplits() const { return (int)in_sizes_.size(); }
  int numOutSplits() const { return (int)out_sizes_.size(); }
  // omega > 0: every tile's weights are divided by max|w_tile| / omega and the quotient becomes
  // the tile's digital output scale (TileWithPeriphery.apply_weight_scaling,
  // src/aihwkit/simulator/tiles/periphery.py:437-500, layer-wise form); omega = 0: scales 1
  void setWeights(const float *w_host, float omega = 0.0f);
  // logical weights: tile weights times their output scales
  void getWeights(float *w_host);
  // digital bias [out_size] added after the sum over in-splits (array.py:178-181); null removes it
  void setBias(const float *bias_host);
  const std::vector<float> &tileScales() const { return tile_scale_host_; }
  void forward(const float *x, float *y, int m, bool is_test, cudaStream_t s);
  // input that holds only the locally owned columns: [m][localInSize()]
  void forwardLocal(const float *x_local, float *y, int m, bool is_test, cudaStream_t s);
  int localInSize() const;
  // Forward of a sharded layer with the partial sums written straight to the owners of the row
  // blocks (reduce-scatter by direct stores): x_local is [m][localInSize()]; owner q receives
  // rows [q * rows_per_owner, (q + 1) * rows_per_owner) at out_table[q] (device array of n_owners
  // pointers into local or peer memory, row pitch out_size). Needs the tensor-core path.
  void forwardScatter(const float *x_local, int m, float *const *out_table_dev, int n_owners,
                      int rows_per_owner, int rotate_rows, cudaStream_t s);
  // the same with signed-byte ADC codes per in-split instead of fp32 sums (see the C header)
  bool scatterCodesSupported();
  void forwardScatterCodes(const float *x_local, int m, uint8_t *const *code_table_dev,
                           float *const *fac_table_dev, int n_owners, int rows_per_owner,
                           int rotate_rows, cudaStream_t s);
  // general form of both (ab200_scatter_plan of the C header): a batch cut into several
  // launches, rows dealt to the owners in blocks, completion flags for the owners
  void forwardScatterPlan(const float *x_local, int m, const ab200_scatter_plan &plan, cudaStream_t s);
  // Training of a mapped layer, tile by tile as autograd does in the reference
  // (TileModuleArray modules -> TileWithPeriphery.backward / update, tiles/periphery.py:1068-1110,
  // 1154-1230). backward: x_grad[:, in-split i] = sum over out-splits o of
  // tile(i, o).backward(d[:, out-split o] * alpha_io); update: tile(i, o).update(x[:, in-split i],
  // d[:, out-split o] / alpha_io). d is [m][out_size]; x / x_grad are [m][in_size] (full width;
  // only the locally owned columns are read / written).
  void backward(const float *d, float *x_grad, int m, cudaStream_t s);
  void update(const float *x, const float *d, int m, cudaStream_t s);
  void setLearningRate(float lr);
  void forwardHost(const float *x, float *y, int m, bool is_test, cudaStream_t s);
  void setSeed(uint64_t seed);

private:
  mutable std::mutex mu_; // held by every C-ABI call on this array
  // in_local / out_local count from in_begin_ / out_begin_
  Tile &tile(int in_local, int out_local) { return *tiles_[(size_t)in_local * nOutLocal() + out_local]; }
  int nOutLocal() const { return out_end_ - out_begin_; }
  bool ownsAllOutSplits() const { return out_begin_ == 0 && out_end_ == (int)out_sizes_.size(); }
  int out_size_, in_size_, device_;
  std::vector<int> in_sizes_, out_sizes_, in_off_, out_off_;
  int in_begin_, in_end_;
  int out_begin_ = 0, out_end_ = 0;
  std::vector<std::unique_ptr<Tile>> tiles_;
  // one tensor-core engine for all locally owned tiles; operands are refreshed per tile when
  // that tile's weights changed
  // digital periphery: output scale per local tile [in_local][out] and bias [out_size]
  std::vector<float> tile_scale_host_;
  float *tile_scale_dev_ = nullptr;
  bool scaled_ = false;
  float *bias_dev_ = nullptr;
  const ab200_scatter_plan *plan_ = nullptr; // set only while a scatter forward runs
  float *d_scratch_ = nullptr; // [m][largest out-split]: gradients times / over the tile scale
  size_t d_scratch_floats_ = 0;
  const float *scaledGradient(const float *d, int oi, int m, float factor, long long &ld,
                              cudaStream_t s, bool divide = false);
  std::unique_ptr<TcEngine> tc_;
  std::vector<uint64_t> tc_versions_;
  bool tcEligible(int m);
  // x0 points at the first locally owned column of row 0, x_ss is the row pitch
  void forwardImpl(const float *x0, long long x_ss, float *y, int m, cudaStream_t s);
  void forwardTc(const float *x0, long long x_ss, float *y, int m, cudaStream_t s);
  // host-buffer path: the batch is cut into row chunks that flow through a three-stage pipeline
  // (host -> device copy, kernels, device -> host copy) on three streams with two buffers each
  static constexpr int kHostChunkRows = 1024;
  float *xd_[2] = {nullptr, nullptr}, *yd_[2] = {nullptr, nullptr};
  float *xh_[2] = {nullptr, nullptr}, *yh_[2] = {nullptr, nullptr}; // pinned staging (pageable callers)
  cudaStream_t s_h2d_ = nullptr, s_d2h_ = nullptr;
  cudaEvent_t ev_h2d_[2] = {nullptr, nullptr}, ev_comp_[2] = {nullptr, nullptr},
              ev_d2h_[2] = {nullptr, nullptr};
  bool host_ready_ = false;
  void ensureHostPipeline();
};

} // namespace ab200
