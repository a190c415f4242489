#include "array.h"

#include <algorithm>
#include <cstring>

namespace ab200 {

// TileModuleArray.get_split_sizes (src/aihwkit/simulator/tiles/array.py:82-97)
std::vector<int> splitSizes(int size, int split_max) {
  if (split_max <= 0) {
    return {size};
  }
  int n = (size + split_max - 1) / split_max;
  int base = size / n, extra = size % n;
  std::vector<int> out(n);
  for (int i = 0; i < n; i++) {
    out[i] = base + (i < extra ? 1 : 0);
  }
  return out;
}

// All tiles of a layer share one noise key; tile (i, o) draws from its own counter stream,
// selected by its GLOBAL index i * n_out + o, so a sharded layer draws the same noise no matter
// how many ranks it is spread over.

TileArray::TileArray(const ab200_tile_config &cfg, int out_size, int in_size, int max_out,
                     int max_in, int in_begin, int in_end, int cuda_device, int out_begin, int out_end)
    : out_size_(out_size), in_size_(in_size), device_(cuda_device) {
  if (out_size <= 0 || in_size <= 0) {
    AB200_FATAL("array sizes must be positive");
  }
  in_sizes_ = splitSizes(in_size, max_in);
  out_sizes_ = splitSizes(out_size, max_out);
  int off = 0;
  for (int v : in_sizes_) {
    in_off_.push_back(off);
    off += v;
  }
  off = 0;
  for (int v : out_sizes_) {
    out_off_.push_back(off);
    off += v;
  }
  if (in_end < 0) {
    in_end = (int)in_sizes_.size();
  }
  if (in_begin < 0 || in_begin > in_end || in_end > (int)in_sizes_.size()) {
    AB200_FATAL("array: invalid in-split range [" << in_begin << ", " << in_end << ")");
  }
  in_begin_ = in_begin;
  in_end_ = in_end;
  if (out_end < 0) {
    out_end = (int)out_sizes_.size();
  }
  if (out_begin < 0 || out_begin > out_end || out_end > (int)out_sizes_.size()) {
    AB200_FATAL("array: invalid out-split range [" << out_begin << ", " << out_end << ")");
  }
  out_begin_ = out_begin;
  out_end_ = out_end;
  uint64_t seed = cfg.seed ? cfg.seed : 0x1234567ull;
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      ab200_tile_config c = cfg;
      c.x_size = in_sizes_[ii];
      c.d_size = out_sizes_[oi];
      c.seed = seed;
      if (c.device[0].construction_seed) {
        c.device[0].construction_seed += (uint32_t)(ii * 4099 + oi);
      }
      tiles_.emplace_back(new Tile(c, cuda_device));
    }
  }
}

TileArray::~TileArray() {
  for (int b = 0; b < 2; b++) {
    cudaFree(xd_[b]);
    cudaFree(yd_[b]);
    cudaFreeHost(xh_[b]);
    cudaFreeHost(yh_[b]);
    if (ev_h2d_[b]) {
      cudaEventDestroy(ev_h2d_[b]);
      cudaEventDestroy(ev_comp_[b]);
      cudaEventDestroy(ev_d2h_[b]);
    }
  }
  if (s_h2d_) {
    cudaStreamDestroy(s_h2d_);
    cudaStreamDestroy(s_d2h_);
  }
  cudaFree(tile_scale_dev_);
  cudaFree(bias_dev_);
  cudaFree(d_scratch_);
}

void TileArray::setSeed(uint64_t seed) {
  for (auto &t : tiles_) {
    t->setSeed(seed ? seed : 0x1234567ull);
  }
}

void TileArray::setWeights(const float *w_host, float omega) {
  std::vector<float> buf;
  const int n_out = nOutLocal();
  tile_scale_host_.assign((size_t)(in_end_ - in_begin_) * n_out, 1.0f);
  scaled_ = omega > 0.0f;
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      int xs = in_sizes_[ii], ds = out_sizes_[oi];
      buf.resize((size_t)xs * ds);
      float amax = 0.0f;
      for (int r = 0; r < ds; r++) {
        const float *src = w_host + (size_t)(out_off_[oi] + r) * in_size_ + in_off_[ii];
        std::memcpy(&buf[(size_t)r * xs], src, (size_t)xs * sizeof(float));
        for (int c = 0; c < xs; c++) {
          amax = std::max(amax, std::fabs(src[c]));
        }
      }
      if (scaled_) {
        float alpha = amax / omega;
        if (alpha == 0.0f) {
          alpha = 1.0f;
        }
        for (float &v : buf) {
          v /= alpha;
        }
        tile_scale_host_[(size_t)(ii - in_begin_) * n_out + (oi - out_begin_)] = alpha;
      }
      tile(ii - in_begin_, oi - out_begin_).setWeights(buf.data());
    }
  }
  if (!tile_scale_host_.empty()) {
    AB200_CUDA(cudaSetDevice(device_));
    if (!tile_scale_dev_) {
      AB200_CUDA(cudaMalloc(&tile_scale_dev_, tile_scale_host_.size() * sizeof(float)));
    }
    AB200_CUDA(cudaMemcpy(tile_scale_dev_, tile_scale_host_.data(),
                          tile_scale_host_.size() * sizeof(float), cudaMemcpyHostToDevice));
  }
}

void TileArray::setBias(const float *bias_host) {
  AB200_CUDA(cudaSetDevice(device_));
  if (!bias_host) {
    cudaFree(bias_dev_);
    bias_dev_ = nullptr;
    return;
  }
  if (!bias_dev_) {
    AB200_CUDA(cudaMalloc(&bias_dev_, (size_t)out_size_ * sizeof(float)));
  }
  AB200_CUDA(cudaMemcpy(bias_dev_, bias_host, (size_t)out_size_ * sizeof(float), cudaMemcpyHostToDevice));
}

void TileArray::getWeights(float *w_host) {
  std::vector<float> buf;
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      int xs = in_sizes_[ii], ds = out_sizes_[oi];
      buf.resize((size_t)xs * ds);
      tile(ii - in_begin_, oi - out_begin_).getWeights(buf.data());
      if (scaled_) {
        const float alpha = tile_scale_host_[(size_t)(ii - in_begin_) * nOutLocal() + (oi - out_begin_)];
        for (float &v : buf) {
          v *= alpha;
        }
      }
      for (int r = 0; r < ds; r++) {
        std::memcpy(w_host + (size_t)(out_off_[oi] + r) * in_size_ + in_off_[ii],
                    &buf[(size_t)r * xs], (size_t)xs * sizeof(float));
      }
    }
  }
}

// digital bias of the layer, for the path that runs the tiles one by one: y[r * ld + c] += bias[c]
// for a block of `cols` columns
__global__ void __launch_bounds__(256)
    addBiasBlockKernel(float *y, long long ld, const float *bias, int cols, long long n) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    const long long r = t / cols;
    const int c = (int)(t - r * cols);
    y[r * ld + c] += bias[c];
  }
}

// TileModuleArray.forward (array.py:155-182): per-tile analog MVM, sum over in-splits after each
// tile's ADC, concatenation over out-splits.
int TileArray::localInSize() const {
  int n = 0;
  for (int ii = in_begin_; ii < in_end_; ii++) {
    n += in_sizes_[ii];
  }
  return n;
}

void TileArray::forward(const float *x, float *y, int m, bool is_test, cudaStream_t s) {
  (void)is_test;
  forwardImpl(in_begin_ < in_end_ ? x + in_off_[in_begin_] : x, in_size_, y, m, s);
}

void TileArray::forwardLocal(const float *x_local, float *y, int m, bool is_test, cudaStream_t s) {
  (void)is_test;
  forwardImpl(x_local, localInSize(), y, m, s);
}

void TileArray::forwardImpl(const float *x0, long long x_ss, float *y, int m, cudaStream_t s) {
  if (m <= 0) {
    return;
  }
  if (in_begin_ == in_end_ || out_begin_ == out_end_) {
    AB200_CUDA(cudaMemsetAsync(y, 0, (size_t)m * out_size_ * sizeof(float), s));
    return;
  }
  if (!ownsAllOutSplits()) {
    // a shard's contribution to the sum over all shards: zero outside its own columns
    AB200_CUDA(cudaMemsetAsync(y, 0, (size_t)m * out_size_ * sizeof(float), s));
  }
  if (tcEligible(m)) {
    forwardTc(x0, x_ss, y, m, s);
    return;
  }
  const int n_out = (int)out_sizes_.size(), n_ol = nOutLocal();
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      const float alpha =
          scaled_ ? tile_scale_host_[(size_t)(ii - in_begin_) * n_ol + (oi - out_begin_)] : 1.0f;
      tile(ii - in_begin_, oi - out_begin_)
          .forwardStrided(x0 + (in_off_[ii] - in_off_[in_begin_]), x_ss, y + out_off_[oi],
                          out_size_, m,
                          /*accumulate=*/ii != in_begin_,
                          (uint32_t)(ii * n_out + oi), alpha, s);
    }
  }
  // the digital bias enters the sum over the shards once: with the shard of the first in-split
  if (bias_dev_ && in_begin_ == 0) {
    const int c0 = out_off_[out_begin_];
    const int cols = (out_end_ < (int)out_sizes_.size() ? out_off_[out_end_] : out_size_) - c0;
    addBiasBlockKernel<<<(unsigned)(((long long)m * cols + 255) / 256), 256, 0, s>>>(
        y + c0, out_size_, bias_dev_ + c0, cols, (long long)m * cols);
    AB200_LAUNCH_CHECK();
  }
}

// dst[r][c] = src[r * src_ld + c] * factor (or / factor): the gradient block of one out-split,
// scaled the way the reference's periphery scales it - a product before the backward pass, a
// quotient before the update (tiles/periphery.py pre_backward / pre_update): the quotient and the
// product with the reciprocal differ in the last bit, which can move a pulse count
__global__ void __launch_bounds__(256)
    scaleBlockKernel(const float *src, long long src_ld, float *dst, int cols, long long n,
                     float factor, int divide) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    const float v = src[(t / cols) * src_ld + t % cols];
    dst[t] = divide ? __fdiv_rn(v, factor) : __fmul_rn(v, factor);
  }
}

const float *TileArray::scaledGradient(const float *d, int oi, int m, float factor, long long &ld,
                                       cudaStream_t s, bool divide) {
  if (factor == 1.0f) {
    ld = out_size_;
    return d + out_off_[oi];
  }
  const int cols = out_sizes_[oi];
  const size_t need = (size_t)m * cols;
  if (need > d_scratch_floats_) {
    AB200_CUDA(cudaStreamSynchronize(s));
    cudaFree(d_scratch_);
    AB200_CUDA(cudaMalloc(&d_scratch_, need * sizeof(float)));
    d_scratch_floats_ = need;
  }
  scaleBlockKernel<<<(unsigned)((need + 255) / 256), 256, 0, s>>>(d + out_off_[oi], out_size_,
                                                               d_scratch_, cols, (long long)need,
                                                               factor, divide ? 1 : 0);
  AB200_LAUNCH_CHECK();
  ld = cols;
  return d_scratch_;
}

void TileArray::forwardScatter(const float *x_local, int m, float *const *out_table_dev,
                               int n_owners, int rows_per_owner, int rotate_rows, cudaStream_t s) {
  ab200_scatter_plan plan{};
  plan.out_table_dev = out_table_dev;
  plan.n_owners = n_owners;
  plan.rows_per_owner = rows_per_owner;
  plan.rotate_rows = rotate_rows;
  forwardScatterPlan(x_local, m, plan, s);
}

bool TileArray::scatterCodesSupported() {
  if (in_begin_ == in_end_ || !ownsAllOutSplits() || scaled_ || bias_dev_ != nullptr ||
      (out_size_ & 31) != 0) {
    return false;
  }
  for (int n : out_sizes_) {
    if ((n % 128) != 0) {
      return false;
    }
  }
  return TcEngine::codesSupported(tiles_[0]->fio());
}

void TileArray::forwardScatterCodes(const float *x_local, int m, uint8_t *const *code_table_dev,
                                    float *const *fac_table_dev, int n_owners, int rows_per_owner,
                                    int rotate_rows, cudaStream_t s) {
  ab200_scatter_plan plan{};
  plan.code_table_dev = code_table_dev;
  plan.fac_table_dev = fac_table_dev;
  plan.n_owners = n_owners;
  plan.rows_per_owner = rows_per_owner;
  plan.rotate_rows = rotate_rows;
  forwardScatterPlan(x_local, m, plan, s);
}

void TileArray::forwardScatterPlan(const float *x_local, int m, const ab200_scatter_plan &plan,
                                   cudaStream_t s) {
  if (m <= 0) {
    return;
  }
  const bool codes = plan.code_table_dev != nullptr;
  if (in_begin_ == in_end_) {
    AB200_FATAL("forward_scatter: this shard owns no in-split");
  }
  if (!ownsAllOutSplits()) {
    AB200_FATAL("forward_scatter: the shard has to own all out-splits of its in-splits");
  }
  if ((plan.out_table_dev != nullptr) == codes) {
    AB200_FATAL("forward_scatter: give either the fp32 buffers or the code and factor buffers");
  }
  if (!tcEligible(m)) {
    AB200_FATAL("forward_scatter needs the tensor-core path (batch >= 128, IO settings with integer "
                "DAC codes, no bound management)");
  }
  if (codes && (!scatterCodesSupported() || plan.fac_table_dev == nullptr)) {
    AB200_FATAL("forward_scatter_codes: this array is not eligible (see "
                "ab200_array_scatter_codes_supported; batch >= 128)");
  }
  if (plan.n_owners <= 0 || plan.rows_per_owner <= 0 || plan.row_base < 0 ||
      (codes && (plan.rows_per_owner & 31) != 0) || plan.owner_block_rows < 0 ||
      (plan.owner_block_rows & 31) != 0 || (plan.row_base & 31) != 0) {
    AB200_FATAL("forward_scatter: invalid owner layout");
  }
  // the last row of the launch has to fit into its owner's buffer
  {
    const long long last = (long long)plan.row_base + m - 1;
    long long lrow;
    if (plan.owner_block_rows > 0) {
      const long long blk = last / plan.owner_block_rows;
      lrow = (blk / plan.n_owners) * plan.owner_block_rows + last % plan.owner_block_rows;
    } else {
      lrow = last - (long long)(plan.n_owners - 1) * plan.rows_per_owner;
    }
    if (lrow >= plan.rows_per_owner) {
      AB200_FATAL("forward_scatter: the owners' row blocks do not cover the batch");
    }
  }
  plan_ = &plan;
  try {
    forwardTc(x_local, localInSize(), nullptr, m, s);
  } catch (...) {
    plan_ = nullptr;
    throw;
  }
  plan_ = nullptr;
}

void TileArray::backward(const float *d, float *x_grad, int m, cudaStream_t s) {
  if (m <= 0) {
    return;
  }
  AB200_CUDA(cudaSetDevice(device_));
  const int n_out = (int)out_sizes_.size(), n_ol = nOutLocal();
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      const float alpha =
          scaled_ ? tile_scale_host_[(size_t)(ii - in_begin_) * n_ol + (oi - out_begin_)] : 1.0f;
      long long ld = 0;
      // pre_backward: the gradient is multiplied by the mapping scale before the tile sees it
      const float *dt = scaledGradient(d, oi, m, alpha, ld, s);
      tile(ii - in_begin_, oi - out_begin_)
          .backwardStrided(dt, ld, x_grad + in_off_[ii], in_size_, m, /*accumulate=*/oi != out_begin_,
                           (uint32_t)(ii * n_out + oi), 1.0f, s);
    }
  }
}

void TileArray::update(const float *x, const float *d, int m, cudaStream_t s) {
  if (m <= 0) {
    return;
  }
  AB200_CUDA(cudaSetDevice(device_));
  const int n_ol = nOutLocal();
  for (int ii = in_begin_; ii < in_end_; ii++) {
    for (int oi = out_begin_; oi < out_end_; oi++) {
      const float alpha =
          scaled_ ? tile_scale_host_[(size_t)(ii - in_begin_) * n_ol + (oi - out_begin_)] : 1.0f;
      long long ld = 0;
      // pre_update: the gradient is divided by the mapping scale
      const float *dt = scaledGradient(d, oi, m, alpha, ld, s, /*divide=*/true);
      tile(ii - in_begin_, oi - out_begin_).updateStrided(x + in_off_[ii], in_size_, dt, ld, m, s);
    }
  }
}

void TileArray::setLearningRate(float lr) {
  for (auto &t : tiles_) {
    t->setLearningRate(lr);
  }
}

bool TileArray::tcEligible(int m) {
  const int mode = mvmPath();
  if (mode == 1 || tiles_.empty()) {
    return false;
  }
  const IOEff &io = tiles_[0]->fio();
  if (!TcEngine::ioSupported(io) || io.bm != AB200_BM_NONE) {
    return false;
  }
  return mode >= 2 || m >= 128;
}

// All local tiles in one launch: the DAC kernel quantises every (row, in-split) once, the MMA
// kernel walks the in-splits per 128 x 128 output block and sums them after each tile's ADC.
void TileArray::forwardTc(const float *x0, long long x_ss, float *y, int m, cudaStream_t s) {
  const int n_in = in_end_ - in_begin_, n_out = nOutLocal(), n_out_total = (int)out_sizes_.size();
  if (!tc_) {
    tc_.reset(new TcEngine(device_));
    tc_->configure(std::vector<int>(in_sizes_.begin() + in_begin_, in_sizes_.begin() + in_end_),
                   std::vector<int>(out_sizes_.begin() + out_begin_, out_sizes_.begin() + out_end_));
    tc_versions_.assign((size_t)n_in * n_out, 0);
  }
  TcEngine::Run r;
  r.key = tile(0, 0).noiseKey();
  // tile (i, o) of the whole layer draws from stream i * n_out_total + o, whatever the shard
  r.noise_id0 = (uint32_t)(in_begin_ * n_out_total + out_begin_);
  r.noise_stride = n_out_total;
  for (int il = 0; il < n_in; il++) {
    for (int oi = 0; oi < n_out; oi++) {
      Tile &t = tile(il, oi);
      const size_t idx = (size_t)il * n_out + oi;
      if (tc_versions_[idx] != t.weightsVersion()) {
        // forward operand: B[n = d][k = x] = w[k * d_size + n]
        tc_->loadOperand(il, oi, t.weightsXD(), t.dSize(), 1, s);
        tc_versions_[idx] = t.weightsVersion();
      }
      // every tile's call counter advances together; the group uses one value
      const uint32_t call = t.nextForwardCall();
      if (idx == 0) {
        r.call = call;
      }
    }
  }
  r.in = x0;
  r.in_ss = x_ss;
  r.m = m;
  const int c0 = out_off_[out_begin_];
  r.out = y ? y + c0 : nullptr;
  r.out_ss = out_size_;
  r.io = tiles_[0]->fio();
  r.tile_scale = scaled_ ? tile_scale_dev_ : nullptr;
  // the digital bias enters the sum over the shards once: with the shard of the first in-split
  r.bias = (bias_dev_ && in_begin_ == 0) ? bias_dev_ + c0 : nullptr;
  if (plan_) {
    r.out_table = plan_->out_table_dev;
    r.code_table = plan_->code_table_dev;
    r.fac_table = plan_->fac_table_dev;
    r.rows_per_owner = plan_->rows_per_owner;
    r.rotate_rows = plan_->rotate_rows;
    r.row_base = plan_->row_base;
    r.n_owners = plan_->n_owners;
    r.owner_block_rows = plan_->owner_block_rows;
    r.flag_table = plan_->flag_table_dev;
    r.epoch = plan_->epoch;
  }
  tc_->run(r, s);
}

void TileArray::ensureHostPipeline() {
  if (host_ready_) {
    return;
  }
  const size_t nx = (size_t)kHostChunkRows * in_size_, ny = (size_t)kHostChunkRows * out_size_;
  for (int b = 0; b < 2; b++) {
    AB200_CUDA(cudaMalloc(&xd_[b], nx * sizeof(float)));
    AB200_CUDA(cudaMalloc(&yd_[b], ny * sizeof(float)));
    AB200_CUDA(cudaMallocHost(&xh_[b], nx * sizeof(float)));
    AB200_CUDA(cudaMallocHost(&yh_[b], ny * sizeof(float)));
    AB200_CUDA(cudaEventCreateWithFlags(&ev_h2d_[b], cudaEventDisableTiming));
    AB200_CUDA(cudaEventCreateWithFlags(&ev_comp_[b], cudaEventDisableTiming));
    AB200_CUDA(cudaEventCreateWithFlags(&ev_d2h_[b], cudaEventDisableTiming));
  }
  AB200_CUDA(cudaStreamCreateWithFlags(&s_h2d_, cudaStreamNonBlocking));
  AB200_CUDA(cudaStreamCreateWithFlags(&s_d2h_, cudaStreamNonBlocking));
  host_ready_ = true;
}

static bool isPinnedHost(const void *p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost;
}

// Host-buffer forward. Copies and kernels of different row chunks overlap: while chunk c is in the
// kernels, chunk c + 1 is on its way to the device and chunk c - 1 on its way back, so the call
// costs about max(copy in, compute, copy out) instead of their sum. Page-locked caller buffers
// (cudaHostRegister / torch pin_memory) are copied directly; pageable ones go through the
// library's own pinned staging buffers.
void TileArray::forwardHost(const float *x, float *y, int m, bool is_test, cudaStream_t s) {
  AB200_CUDA(cudaSetDevice(device_));
  if (m <= 0) {
    return;
  }
  ensureHostPipeline();
  const bool x_pinned = isPinnedHost(x), y_pinned = isPinnedHost(y);
  const int R = kHostChunkRows;
  const int n_chunks = (m + R - 1) / R;
  // the caller's stream may have earlier work that produced x or must precede our kernels
  for (int c = 0; c < n_chunks; c++) {
    const int b = c & 1;
    const int rows = std::min(R, m - c * R);
    const size_t nx = (size_t)rows * in_size_, ny = (size_t)rows * out_size_;
    const float *xc = x + (size_t)c * R * in_size_;
    float *yc = y + (size_t)c * R * out_size_;
    // input buffer b is free once the kernels of chunk c - 2 are done
    if (c >= 2) {
      AB200_CUDA(cudaStreamWaitEvent(s_h2d_, ev_comp_[b], 0));
    }
    if (x_pinned) {
      AB200_CUDA(cudaMemcpyAsync(xd_[b], xc, nx * sizeof(float), cudaMemcpyHostToDevice, s_h2d_));
    } else {
      if (c >= 2) {
        AB200_CUDA(cudaEventSynchronize(ev_h2d_[b])); // staging buffer b has left the host
      }
      std::memcpy(xh_[b], xc, nx * sizeof(float));
      AB200_CUDA(cudaMemcpyAsync(xd_[b], xh_[b], nx * sizeof(float), cudaMemcpyHostToDevice, s_h2d_));
    }
    AB200_CUDA(cudaEventRecord(ev_h2d_[b], s_h2d_));
    // kernels: need the input, and output buffer b drained (copy-out of chunk c - 2)
    AB200_CUDA(cudaStreamWaitEvent(s, ev_h2d_[b], 0));
    if (c >= 2) {
      AB200_CUDA(cudaStreamWaitEvent(s, ev_d2h_[b], 0));
    }
    forward(xd_[b], yd_[b], rows, is_test, s);
    AB200_CUDA(cudaEventRecord(ev_comp_[b], s));
    // copy-out
    AB200_CUDA(cudaStreamWaitEvent(s_d2h_, ev_comp_[b], 0));
    if (y_pinned) {
      AB200_CUDA(cudaMemcpyAsync(yc, yd_[b], ny * sizeof(float), cudaMemcpyDeviceToHost, s_d2h_));
      AB200_CUDA(cudaEventRecord(ev_d2h_[b], s_d2h_));
    } else {
      if (c >= 2) {
        // the previous use of staging buffer b must reach the caller's memory first
        AB200_CUDA(cudaEventSynchronize(ev_d2h_[b]));
        const int pc = c - 2;
        const int prows = std::min(R, m - pc * R);
        std::memcpy(y + (size_t)pc * R * out_size_, yh_[b], (size_t)prows * out_size_ * sizeof(float));
      }
      AB200_CUDA(cudaMemcpyAsync(yh_[b], yd_[b], ny * sizeof(float), cudaMemcpyDeviceToHost, s_d2h_));
      AB200_CUDA(cudaEventRecord(ev_d2h_[b], s_d2h_));
    }
  }
  AB200_CUDA(cudaStreamSynchronize(s_d2h_));
  AB200_CUDA(cudaStreamSynchronize(s));
  if (!y_pinned) {
    for (int pc = std::max(0, n_chunks - 2); pc < n_chunks; pc++) {
      const int prows = std::min(R, m - pc * R);
      std::memcpy(y + (size_t)pc * R * out_size_, yh_[pc & 1], (size_t)prows * out_size_ * sizeof(float));
    }
  }
}

} // namespace ab200
