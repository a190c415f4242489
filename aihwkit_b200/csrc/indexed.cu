// Indexed (im2col-free) convolution interface of the analog tile: the caller hands over whole
// images and an index array that says, for every tile input and every output position, which
// image element feeds it (0 = padding, 1 = the constant of an analog bias, j >= 2 = element j - 2).
// Reference: RPUSimple<T>::copyIndexedInput / copyIndexedOutput / forwardIndexed / backwardIndexed /
// updateIndexed (src/rpucuda/rpu.cpp:846-1013, 1117-1239); the reference GPU reads through
// iterators instead (src/rpucuda/cuda/io_iterator.h:194-303).
//
// Here the forward pass on the tensor-core path and the pulsed update read the images through
// the index array themselves (the DAC kernel and the pulse-preparation kernel gather a row each,
// RowGather in tile.h), so the unfolded matrix is never written; other cases (CUDA-core MVM,
// floating-point update) go through the sample-major matrix [dim3 * m_batch][x_size] (row = one
// output position of one image). The MVM kernels store image-major outputs
// [dim3][d_size][m_batch] themselves (MvmProblem::out_t_rows). The backward pass stores the input
// gradients of all positions in the layout of the index array, and every image element then sums
// the positions that name it through an inverse index built once per index array: no atomics,
// and the same bits on every run.
#include "tile.h"

#include <cstdlib>
#include <vector>

namespace ab200 {

namespace {

// cols[(n * m_batch + l) * size + r] = src(n, idx[r][l]);  idx is [size][m_batch]
// Tile of 32 positions x 32 inputs through shared memory: the index array and the image are read
// along l (neighbouring output positions read neighbouring pixels), the matrix is written along r.
__global__ void __launch_bounds__(256)
    gatherTransKernel(const float *x, const int *idx, float *cols, int size, int m_batch,
                      long long in_mat) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int l0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const float *img = x + (long long)n * in_mat;
  for (int k = threadIdx.y; k < 32; k += 8) {
    const int r = r0 + k, l = l0 + threadIdx.x;
    float v = 0.0f;
    if (r < size && l < m_batch) {
      const int j = idx[(long long)r * m_batch + l];
      v = j <= 1 ? (float)j : img[j - 2];
    }
    tile[k][threadIdx.x] = v;
  }
  __syncthreads();
  for (int k = threadIdx.y; k < 32; k += 8) {
    const int l = l0 + k, r = r0 + threadIdx.x;
    if (r < size && l < m_batch) {
      cols[((long long)n * m_batch + l) * size + r] = tile[threadIdx.x][k];
    }
  }
}

// idx is [m_batch][size]: the matrix and the index array have the same order
__global__ void __launch_bounds__(256)
    gatherPlainKernel(const float *x, const int *idx, float *cols, long long per_image,
                      long long in_mat) {
  const int n = blockIdx.y;
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < per_image) {
    const int j = idx[t];
    cols[n * per_image + t] = j <= 1 ? (float)j : x[n * in_mat + j - 2];
  }
}

// out(n, e) = sum over the positions t of the index array that name element e of cols[n][t], in
// ascending t: the backward pass of the indexed interface as a gather, without atomics and with a
// fixed summation order. `cols` has the layout of the index array per image. Neighbouring
// elements are named by neighbouring positions (same kernel tap, next output position), so the
// reads of a warp are contiguous where the index array is [x_size][m_batch].
__global__ void __launch_bounds__(256)
    gatherSumKernel(const float *cols, const int *csr_off, const int *csr_pos, float *out,
                    long long csr_elems, long long out_mat, long long per_image) {
  const int n = blockIdx.y;
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= out_mat) {
    return;
  }
  float acc = 0.0f;
  if (e < csr_elems) {
    const float *c = cols + n * per_image;
    const int t1 = csr_off[e + 1];
    for (int t = csr_off[e]; t < t1; t++) {
      acc += c[csr_pos[t]];
    }
  }
  out[n * out_mat + e] = acc;
}

// dst[b][c][r] = src[b][r][c]
__global__ void __launch_bounds__(256)
    batchedTransposeKernel(const float *src, float *dst, int rows, int cols) {
  __shared__ float tile[32][33];
  const long long base = (long long)blockIdx.z * rows * cols;
  const int c = blockIdx.x * 32 + threadIdx.x, r = blockIdx.y * 32 + threadIdx.y;
  for (int k = 0; k < 32; k += 8) {
    if (c < cols && r + k < rows) {
      tile[threadIdx.y + k][threadIdx.x] = src[base + (long long)(r + k) * cols + c];
    }
  }
  __syncthreads();
  const int oc = blockIdx.y * 32 + threadIdx.x, orow = blockIdx.x * 32 + threadIdx.y;
  for (int k = 0; k < 32; k += 8) {
    if (oc < rows && orow + k < cols) {
      dst[base + (long long)(orow + k) * rows + oc] = tile[threadIdx.x][threadIdx.y + k];
    }
  }
}

void launchBatchedTranspose(const float *src, float *dst, int rows, int cols, int batch,
                            cudaStream_t s) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
  batchedTransposeKernel<<<grid, block, 0, s>>>(src, dst, rows, cols);
  AB200_LAUNCH_CHECK();
}

} // namespace

void Tile::setMatrixIndices(const int32_t *indices, long long n, cudaStream_t s) {
  requireDevice("set_matrix_indices");
  if (n <= 0 || indices == nullptr) {
    AB200_FATAL("set_matrix_indices: empty index array");
  }
  AB200_CUDA(cudaSetDevice(device_));
  if (n > idx_cap_) {
    if (idx_) {
      AB200_CUDA(cudaFree(idx_));
      idx_ = nullptr;
    }
    AB200_CUDA(cudaMalloc(&idx_, (size_t)n * sizeof(int32_t)));
    idx_cap_ = n;
  }
  // the array may live on the host or on a device; keep an own copy and learn its value range
  // once, so that every later call can reject images that are too small for it on the host
  std::vector<int32_t> host((size_t)n);
  AB200_CUDA(cudaMemcpyAsync(idx_, indices, (size_t)n * sizeof(int32_t), cudaMemcpyDefault, s));
  AB200_CUDA(cudaMemcpyAsync(host.data(), idx_, (size_t)n * sizeof(int32_t),
                             cudaMemcpyDeviceToHost, s));
  AB200_CUDA(cudaStreamSynchronize(s));
  int32_t lo = host[0], hi = host[0];
  for (long long k = 1; k < n; k++) {
    lo = host[k] < lo ? host[k] : lo;
    hi = host[k] > hi ? host[k] : hi;
  }
  if (lo < 0) {
    idx_count_ = 0;
    AB200_FATAL("set_matrix_indices: negative index " << lo);
  }
  idx_count_ = n;
  idx_max_ = hi;
  idx_t_valid_ = false;
  // inverse index (counting sort by image element; positions stay in ascending order)
  csr_elems_ = hi >= 2 ? (long long)hi - 1 : 0;
  std::vector<int32_t> off((size_t)csr_elems_ + 1, 0), pos;
  for (long long k = 0; k < n; k++) {
    if (host[k] >= 2) {
      off[(size_t)host[k] - 1]++; // element e = host[k] - 2 counts into off[e + 1]
    }
  }
  for (long long e = 0; e < csr_elems_; e++) {
    off[(size_t)e + 1] += off[(size_t)e];
  }
  pos.resize((size_t)off[(size_t)csr_elems_]);
  {
    std::vector<int32_t> fill(off.begin(), off.end() - 1);
    for (long long k = 0; k < n; k++) {
      if (host[k] >= 2) {
        pos[(size_t)fill[(size_t)host[k] - 2]++] = (int32_t)k;
      }
    }
  }
  AB200_CUDA(cudaDeviceSynchronize()); // an earlier backward pass may still read the old arrays
  cudaFree(csr_off_);
  cudaFree(csr_pos_);
  csr_off_ = csr_pos_ = nullptr;
  AB200_CUDA(cudaMalloc(&csr_off_, off.size() * sizeof(int32_t)));
  AB200_CUDA(cudaMalloc(&csr_pos_, (pos.empty() ? 1 : pos.size()) * sizeof(int32_t)));
  AB200_CUDA(cudaMemcpy(csr_off_, off.data(), off.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  if (!pos.empty()) {
    AB200_CUDA(cudaMemcpy(csr_pos_, pos.data(), pos.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  }
}

void Tile::requireIndices(const char *what, long long image_size, int m_batch, int n_img) const {
  if (idx_count_ == 0) {
    AB200_FATAL("Matrix indices not set yet!"); // rpu.h:457-463
  }
  if (m_batch <= 0 || n_img <= 0) {
    AB200_FATAL(what << ": m_batch and dim3 must be positive");
  }
  if (idx_count_ != (long long)x_size_ * m_batch) {
    AB200_FATAL(what << ": the index array has " << idx_count_ << " entries, expected x_size * m_batch = "
                     << (long long)x_size_ * m_batch);
  }
  if ((long long)idx_max_ - 2 >= image_size) {
    AB200_FATAL(what << ": index " << idx_max_ << " points outside an image of " << image_size
                     << " elements");
  }
  if (n_img > 65535) {
    AB200_FATAL(what << ": more than 65535 images per call are not supported");
  }
}

void Tile::ensureIndexedScratch(long long b, bool need_x, bool need_d) {
  if (need_x && b > cols_x_cap_) {
    if (cols_x_) {
      AB200_CUDA(cudaDeviceSynchronize());
      AB200_CUDA(cudaFree(cols_x_));
      cols_x_ = nullptr;
    }
    AB200_CUDA(cudaMalloc(&cols_x_, (size_t)b * x_size_ * sizeof(float)));
    cols_x_cap_ = b;
  }
  if (need_d && b > cols_d_cap_) {
    if (cols_d_) {
      AB200_CUDA(cudaDeviceSynchronize());
      AB200_CUDA(cudaFree(cols_d_));
      cols_d_ = nullptr;
    }
    AB200_CUDA(cudaMalloc(&cols_d_, (size_t)b * d_size_ * sizeof(float)));
    cols_d_cap_ = b;
  }
}

const int32_t *Tile::rowMajorIndices(int m_batch, bool trans, cudaStream_t s) {
  if (!trans) {
    return idx_; // already [m_batch][x_size]
  }
  if (!idx_t_valid_) {
    if (idx_count_ > idx_t_cap_) {
      if (idx_t_) {
        AB200_CUDA(cudaDeviceSynchronize());
        AB200_CUDA(cudaFree(idx_t_));
        idx_t_ = nullptr;
      }
      AB200_CUDA(cudaMalloc(&idx_t_, (size_t)idx_count_ * sizeof(int32_t)));
      idx_t_cap_ = idx_count_;
    }
    // [x_size][m_batch] -> [m_batch][x_size]; the entries are moved as 32-bit words
    launchBatchedTranspose(reinterpret_cast<const float *>(idx_), reinterpret_cast<float *>(idx_t_), x_size_,
                           m_batch, 1, s);
    idx_t_valid_ = true;
  }
  return idx_t_;
}

bool Tile::updateGatherEligible() const {
  static const bool off = [] {
    const char *e = getenv("AB200_INDEXED_GATHER");
    return e && e[0] == '0';
  }();
  // the pulse-preparation kernel is the only reader of x on the pulsed path
  // (the mixed-precision compound quantises and accumulates x digitally: it takes the matrix)
  return !off && cfg_.device_kind != AB200_DEVICE_IDEAL && up_.pulse_type != AB200_PULSE_NONE &&
         up_.pulse_type != AB200_PULSE_NONE_WITH_DEVICE && delta_w_ == nullptr && !cfg_.mixed.enabled;
}

void Tile::gatherIndexed(const float *x, long long in_mat, int m_batch, int n_img, bool trans,
                         cudaStream_t s) {
  if (trans) {
    dim3 grid((m_batch + 31) / 32, (x_size_ + 31) / 32, n_img), block(32, 8);
    gatherTransKernel<<<grid, block, 0, s>>>(x, idx_, cols_x_, x_size_, m_batch, in_mat);
  } else {
    const long long per_image = (long long)m_batch * x_size_;
    dim3 grid((unsigned)((per_image + 255) / 256), n_img);
    gatherPlainKernel<<<grid, 256, 0, s>>>(x, idx_, cols_x_, per_image, in_mat);
  }
  AB200_LAUNCH_CHECK();
}

void Tile::forwardIndexed(const float *x, float *d, long long total_input_size, int m_batch,
                          int n_img, bool trans, bool is_test, cudaStream_t s) {
  requireDevice("forward_indexed");
  const long long in_mat = n_img > 0 ? total_input_size / n_img : 0;
  requireIndices("forward_indexed", in_mat, m_batch, n_img);
  const long long b = (long long)m_batch * n_img;
  if (b > 0x7fffffffLL) {
    AB200_FATAL("forward_indexed: m_batch * dim3 does not fit an int");
  }
  const bool fused = forwardGatherEligible((int)b);
  ensureIndexedScratch(b, !fused, false);
  // image-major outputs [dim3][d_size][m_batch] are stored by the MVM kernels themselves
  const int out_t_rows = trans ? m_batch : 0;
  if (fused) {
    RowGather g;
    g.idx = rowMajorIndices(m_batch, trans, s);
    g.m_batch = m_batch;
    g.ld = x_size_;
    g.image_size = in_mat;
    forwardGathered(x, g, d, (int)b, is_test, s, out_t_rows);
  } else {
    gatherIndexed(x, in_mat, m_batch, n_img, trans, s);
    forward(cols_x_, d, false, (int)b, false, false, is_test, s, out_t_rows);
  }
}

void Tile::backwardIndexed(const float *d, float *x, long long total_output_size, int m_batch,
                           int n_img, bool trans, cudaStream_t s) {
  requireDevice("backward_indexed");
  const long long out_mat = n_img > 0 ? total_output_size / n_img : 0;
  requireIndices("backward_indexed", out_mat, m_batch, n_img);
  const long long b = (long long)m_batch * n_img;
  if (b > 0x7fffffffLL) {
    AB200_FATAL("backward_indexed: m_batch * dim3 does not fit an int");
  }
  ensureIndexedScratch(b, true, trans);
  const float *src = d;
  if (trans) {
    launchBatchedTranspose(d, cols_d_, d_size_, m_batch, n_img, s); // -> [dim3][m_batch][d_size]
    src = cols_d_;
  }
  // the input gradients of all positions in the layout of the index array ([x_size][m_batch] per
  // image: stored transposed by the MVM kernels), then every image element sums the positions
  // that name it
  backwardCore(src, d_size_, 1, cols_x_, x_size_, 1, x_size_, (int)b, false, 0, 1.0f, s, trans ? m_batch : 0);
  const long long per_image = (long long)m_batch * x_size_;
  dim3 grid((unsigned)((out_mat + 255) / 256), n_img);
  gatherSumKernel<<<grid, 256, 0, s>>>(cols_x_, csr_off_, csr_pos_, x, csr_elems_, out_mat, per_image);
  AB200_LAUNCH_CHECK();
}

void Tile::updateIndexed(const float *x, const float *d, long long total_input_size, int m_batch,
                         int n_img, bool trans, cudaStream_t s) {
  requireDevice("update_indexed");
  const long long in_mat = n_img > 0 ? total_input_size / n_img : 0;
  requireIndices("update_indexed", in_mat, m_batch, n_img);
  const long long b = (long long)m_batch * n_img;
  if (b > 0x7fffffffLL) {
    AB200_FATAL("update_indexed: m_batch * dim3 does not fit an int");
  }
  const bool fused = updateGatherEligible();
  ensureIndexedScratch(b, !fused, trans);
  const float *src = d;
  if (trans) {
    launchBatchedTranspose(d, cols_d_, d_size_, m_batch, n_img, s);
    src = cols_d_;
  }
  if (fused) {
    upd_gather_.idx = rowMajorIndices(m_batch, trans, s);
    upd_gather_.m_batch = m_batch;
    upd_gather_.ld = x_size_;
    upd_gather_.image_size = in_mat;
    try {
      update(x, src, false, (int)b, false, false, s);
    } catch (...) {
      upd_gather_ = RowGather{};
      throw;
    }
    upd_gather_ = RowGather{};
  } else {
    gatherIndexed(x, in_mat, m_batch, n_img, trans, s);
    update(cols_x_, src, false, (int)b, false, false, s);
  }
}

} // namespace ab200
