// Tensor-core engine of the IO-managed MVM: tcgen05 MMAs with TMEM accumulators, operands staged
// in shared memory by TMA, DAC codes x split-bf16 weights.
//
// One engine serves a group of physical tiles that form a logical layer:
//     out[m][N_total] = sum over in-splits i of  IO_i( codes_i[m][K_i] * W_i[K_i][N_total] )
// where IO_i is the per-tile noise / ADC / clip / rescale of the reference
// (src/rpucuda/rpu_forward_backward_pass.cpp:673-719, 985-987) applied to each in-split's product
// before the sum (TileModuleArray.forward, src/aihwkit/simulator/tiles/array.py:155-182).
// A single tile is the group I = O = 1; backward uses the transposed operand.
#pragma once

#include "tile.h"

#include <vector>

namespace ab200 {

class TcEngine {
public:
  explicit TcEngine(int device);
  ~TcEngine();
  TcEngine(const TcEngine &) = delete;
  TcEngine &operator=(const TcEngine &) = delete;

  // in_sizes[i] = K_i, out_sizes[o] = N_o
  void configure(const std::vector<int> &in_sizes, const std::vector<int> &out_sizes);
  // operand of tile (i, o):  B[n][k] = w[k * wk + n * wn],  stored as bf16 hi + lo
  void loadOperand(int i, int o, const float *w, long long wk, long long wn, cudaStream_t s);

  struct Run {
    const float *in = nullptr; // [m][*], row stride in_ss, in-split i starts at column in_off[i]
    long long in_ss = 0;
    // rows gathered from whole images at `in` (indexed convolution interface) instead
    RowGather gather;
    // std-dev of the output noise of every output line (out_noise_std > 0; single tile), or null
    const float *onv = nullptr;
    int m = 0;
    float *out = nullptr; // [m][N_total], row stride out_ss
    long long out_ss = 0;
    // > 0: stored transposed in blocks of that many rows instead, [m / out_t_rows][N_total][out_t_rows]
    // with out_ss = N_total (image-major layout of the indexed convolution interface)
    int out_t_rows = 0;
    bool accumulate = false;
    bool backward = false;
    IOEff io;
    float alpha = 1.0f;
    // noise: one key and call counter for the whole group; tile (i, o) draws from the stream
    // with purpose tag + noise_id0 + i * O + o, so tiles are independent and the result does
    // not depend on how a layer is split over engines
    PhiloxKey key{0, 0};
    uint32_t call = 0;
    uint32_t noise_id0 = 0;
    // tile (i, o) of this engine draws from stream noise_id0 + i * noise_stride + o; 0 = the
    // engine's own number of out-splits (an engine that holds a block of a larger layer passes
    // the layer's)
    int noise_stride = 0;
    // optional digital periphery of a mapped layer (device pointers): one scale per tile,
    // [I][O], applied to that tile's output before the sum over in-splits, and a bias per output
    // column added once
    const float *tile_scale = nullptr;
    const float *bias = nullptr;
    // optional scatter of the output rows (sharded layer): device array of buffer pointers, one
    // per row-block owner (local or peer memory); row r goes to out_table[r / rows_per_owner] at
    // row r % rows_per_owner with pitch out_ss. rotate_rows (a multiple of the work-item height)
    // is the row the sweep over the row blocks starts at: it staggers the ranks' sweeps so that no
    // owner receives from two ranks at once.
    float *const *out_table = nullptr;
    // codes variant of the scatter (needs codesSupported, out-splits that are multiples of 128,
    // no tile scales / bias): the signed-byte ADC code of every in-split goes to plane i of
    // code_table[owner] in 32 x 32 blocks of 1 KB, the per-row factors to fac_table[owner] as
    // [in-split][row]; `out` is not written
    uint8_t *const *code_table = nullptr;
    float *const *fac_table = nullptr;
    int rows_per_owner = 0;
    int rotate_rows = 0;
    // scatter of a batch that is cut into several launches, or dealt to the owners in blocks:
    // row_base = row of the whole batch this launch starts at; owner_block_rows > 0: blocks of
    // that many rows go to the owners in turn; flag_table (device array, one address per owner,
    // local or peer memory) receives `epoch` when every store of the launch has been issued and
    // fenced at system scope
    int row_base = 0;
    int n_owners = 0;
    int owner_block_rows = 0;
    int *const *flag_table = nullptr;
    int epoch = 0;
    // optional caller-owned per-row scratch (only valid for I == 1): lets the bound-management
    // re-run kernel see the same noise-management values and flags
    float *scale = nullptr, *factor = nullptr, *vnorm = nullptr, *sval = nullptr;
    int *flags = nullptr;
  };
  void run(const Run &r, cudaStream_t s);

  // whether the IO settings can be expressed as integer DAC codes in bf16
  // (`line_table`: the caller passes the std-dev of the output noise of every line, Run::onv)
  static bool ioSupported(const IOEff &io, bool line_table = false);
  // whether rows of this engine's width can be gathered through an index array by the DAC pass
  // (its shared-memory staging of one row per warp must fit)
  static bool gatherSupported(int in_size);
  // whether, in addition, every in-split's result can leave the kernel as signed-byte ADC codes
  static bool codesSupported(const IOEff &io);
  // throws if an earlier launch reported a device-side failure (timeout of a bounded wait)
  void checkStatus();

  int numIn() const { return (int)in_sizes_.size(); }
  int numOut() const { return (int)out_sizes_.size(); }

private:
  struct PartScratch;
  void ensureBatch(int m);
  PartScratch partScratch(const Run &r, int row0);
  // noise management + DAC / MMA kernel for the rows [row0, row0 + rows) of a run
  void launchDac(const Run &r, int row0, int rows, cudaStream_t s);
  void launchMma(const Run &r, int row0, int rows, cudaStream_t s);

  int n_sm_ = 0;
  unsigned smem_raised_ = 0; // kernel variants whose shared-memory limit is set
  size_t gather_smem_raised_ = 0; // shared-memory limit set for the gathering DAC kernel
  int device_;
  std::vector<int> in_sizes_, out_sizes_, in_off_, out_off_;
  int kpad_ = 0;      // padded K of every in-split (multiple of 64)
  int n_chunks_ = 0;  // 128-column chunks over all out-splits
  int nrows_pad_ = 0; // n_chunks_ * 128
  void *op_hi_ = nullptr, *op_lo_ = nullptr; // bf16 [I * nrows_pad][kpad]
  void *codes_ = nullptr;                    // bf16 [m_cap][I * kpad]
  int m_cap_ = 0;
  float *scale_ = nullptr, *factor_ = nullptr, *vnorm_ = nullptr, *sval_ = nullptr;
  int *flags_ = nullptr;
  int *done_ctr_ = nullptr; // finished CTAs of a scatter launch that signals its completion
  int *chunk_tab_ = nullptr;   // int4 per chunk
  int *insplit_tab_ = nullptr; // int4 per in-split
  int *outn_tab_ = nullptr;    // N_o per out-split
  // side stream on which the DAC kernel of a batch's second half overlaps the MMA kernel of the first
  cudaStream_t side_ = nullptr;
  cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
  int *status_host_ = nullptr; // mapped pinned word written by the kernel on failure
  int *status_dev_ = nullptr;
};

} // namespace ab200
