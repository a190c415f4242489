// Tensor-core IO-managed MVM for sm_100a.
//
//   dacQuantizeKernel   noise management + DAC per (row, in-split): abs-max, scale, integer code
//                       (exact in bf16), per-row scale / factor / ||v||.
//   splitWeightsKernel  fp32 weight -> bf16 hi + bf16 lo (hi + lo keeps 16 mantissa bits), laid
//                       out K-major for the MMA B operand.
//   mvmTcKernel         persistent, warp-specialised: one TMA producer thread stages the codes and
//                       the weight operand in shared memory, hi and lo stacked as one 256-row B
//                       tile, so a single tcgen05.mma (M 128, N 256, K 16) per K step yields the
//                       hi product in accumulator columns 0..127 and the lo product in columns
//                       128..255 while reading the codes once; one thread issues the MMAs;
//                       sixteen epilogue warps. TMEM holds two such 256-column accumulators, so
//                       the epilogue of in-split i (TMEM -> registers, hi + lo, Philox noise, ADC,
//                       clip, bound flag, rescale, running sum over the in-splits in registers)
//                       overlaps the MMAs of in-split i + 1. Every wait is bounded; on a time-out
//                       the kernel records a status code, lets its copies land, frees TMEM and
//                       returns.
//
// Element-wise semantics are the helpers of mvm_common.cuh, shared with the CUDA-core path, and
// the noise counters are the same, so both paths produce the same noise for the same call.
#include "mvm_common.cuh"
#include "tc_engine.h"

#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace ab200 {

constexpr int TC_M = 128;      // rows per CTA
constexpr int TC_N = 128;      // output columns per CTA (one chunk)
constexpr int TC_K = 64;       // K elements per chunk (128 B of bf16: one swizzle row)
// K chunks (of TC_K) per pipeline stage: one barrier round trip of the producer and of the MMA
// issuer moves this many chunks. Two chunks per stage measured 5 % faster than one at the same
// bytes in flight; the ring depth itself (4, 6 or 7 chunks) made no difference.
constexpr int TC_KCH = 2;
constexpr int TC_STAGES = 2;
constexpr int TC_STAGE_A = TC_M * TC_K * 2;
constexpr int TC_STAGE_B = TC_N * TC_K * 2;
constexpr int TC_CHUNK_BYTES = TC_STAGE_A + 2 * TC_STAGE_B; // A, then B hi and B lo back to back
constexpr int TC_STAGE_BYTES = TC_KCH * TC_CHUNK_BYTES;
constexpr int TC_ACC_COLS = 2 * TC_N; // hi and lo halves of one accumulator
constexpr int TC_ACC_STAGES = 512 / TC_ACC_COLS;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 2048;
constexpr int TC_EPI_WARPS = 16; // four per TMEM lane quarter, 32 columns each
constexpr int TC_EPI_COLS = TC_N / (TC_EPI_WARPS / 4);
// warps 0..15 epilogue (warp id % 4 = TMEM lane quarter), warp 16 TMA, warp 17 MMA issuer + TMEM
// owner
constexpr int TC_WARP_TMA = TC_EPI_WARPS;
constexpr int TC_WARP_MMA = TC_EPI_WARPS + 1;
constexpr int TC_THREADS = (TC_EPI_WARPS + 2) * 32;
constexpr unsigned long long TC_WAIT_CYCLES = 4000000000ull; // about 2 s at 2 GHz
// CTA-pair variant (cta_group::2): every CTA of a pair stages its own 128 rows of codes and ONE
// half of the stacked weight tile (rank 0 the hi rows, rank 1 the lo rows), so a chunk is 32 KB
constexpr int TC2_KCH = 2;
constexpr int TC2_STAGES = 3;
constexpr int TC2_CHUNK_BYTES = TC_STAGE_A + TC_STAGE_B;
constexpr int TC2_STAGE_BYTES = TC2_KCH * TC2_CHUNK_BYTES;
constexpr int TC2_SMEM_BYTES = TC2_STAGES * TC2_STAGE_BYTES + 2048;

enum : int {
  TC_ERR_FULL = 1,
  TC_ERR_EMPTY = 2,
  TC_ERR_TMEM_FULL = 3,
  TC_ERR_TMEM_EMPTY = 4
};

struct TcKernelParams {
  int m, I, O, n_chunks, nrows_pad, kpad;
  int noise_stride; // tile (i, o) draws from noise stream noise_id0 + i * noise_stride + o
  int group; // chunks per group of the work-item order
  const int4 *chunk;   // {o, n_local0, n_global0, valid}
  const int4 *insplit; // {k0 (code column), n_k_stages, K_i, in_off}
  const int *outn;     // N_o
  PhiloxKey key;
  uint32_t call, noise_id0;
  const float *scale, *factor, *vnorm;
  const float *tile_scale; // [I][O] or null
  const float *bias;       // [N_total] or null
  int *flags;
  float *out;
  long long out_ss;
  // optional scatter of the output rows over several buffers (the row-block owners of a
  // sharded layer, local or peer memory): row r goes to out_table[r / rows_per_owner] at row
  // r % rows_per_owner; null = everything to `out`
  float *const *out_table;
  // codes variant of the scatter: instead of the fp32 sum over this launch's in-splits, the ADC
  // code (one signed byte) of every in-split goes to the owner, plane i of this rank's slot, in
  // blocks of 32 rows x 32 columns (1 KB, row-major); the per-row factors go to fac_table[owner]
  // as [in-split][row]. The owner multiplies and sums (codeSlotsKernel).
  uint8_t *const *code_table;
  float *const *fac_table;
  int rows_per_owner;
  int rb_rotate; // the sweep over the row blocks starts at this block (staggers the ranks)
  // row of the whole batch this launch starts at (a batch may be cut into several launches):
  // the noise counters and the owner of a scattered row use the row of the whole batch, so the
  // cut does not change the result
  int row_base;
  // scatter: number of owners; owner_blk > 0 deals blocks of that many rows to the owners in
  // turn (block b of the batch is block b / n_owners of owner b % n_owners) instead of giving
  // owner q the rows [q * rows_per_owner, (q + 1) * rows_per_owner)
  int n_owners, owner_blk;
  // optional completion signal of a scatter launch: the last CTA to finish writes `epoch` to
  // flag_table[q] for every owner q (system scope, after every CTA's stores); done_ctr counts
  // the finished CTAs of the launch and is left at zero
  int *const *flag_table;
  int *done_ctr;
  int epoch;
  int accumulate, backward;
  // plain (not scattered) output written the way the scatter writes it: every warp transposes its
  // 32 x 32 block in registers and each store instruction writes 128 contiguous bytes of one
  // row, instead of 16 bytes in each of 32 rows - for outputs so wide that the stores bound the
  // kernel
  int row_stores;
  // std-dev of the output noise per output line ([N_total], single tile; LINE variants), or null
  const float *onv;
  // > 0: the output is stored transposed in blocks of that many rows: row r, column c goes to
  // out[((r / out_t_rows) * out_ss + c) * out_t_rows + r % out_t_rows] (out_ss = columns of the
  // whole layer) - the image-major layout of the indexed convolution interface. The row-per-lane
  // layout of the accumulators is already the right one: every store instruction writes 128
  // contiguous bytes of one column.
  int out_t_rows;
  IOEff io;
  int *status;
  // optional per-CTA cycle counters of time spent waiting, by role (diagnostics; null = off):
  // [0] MMA on operands, [1] MMA issuing instructions, [2] MMA on a free accumulator, [3] MMA
  // total, [4] TMA producer on a free stage, [5] TMA producer issuing copies, [6] epilogue on a
  // complete accumulator, [7] epilogue total
  long long *prof;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarArrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarTry(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(smemAddr(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// bounded wait: false after TC_WAIT_CYCLES or when another role already gave up
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  if (mbarTry(bar, parity)) {
    return true;
  }
  const long long t0 = clock64();
  unsigned spins = 0;
  while (!mbarTry(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*abort_flag != 0 || (unsigned long long)(clock64() - t0) > TC_WAIT_CYCLES) {
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tmaLoad2d(void *dst, const CUtensorMap *map, uint64_t *bar, int x,
                                          int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes"
               " [%0], [%1, {%3, %4}], [%2];" ::"r"(smemAddr(dst)),
               "l"((uint64_t)map), "r"(smemAddr(bar)), "r"(x), "r"(y)
               : "memory");
}
// ---- CTA pairs ----
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapaShared(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbarArriveCluster(uint32_t cluster_addr) {
  // default semantics (release at CTA scope): the TMEM reads this arrive publishes were completed
  // by tcgen05.wait::ld and fenced; a cluster-scope release would also wait for the warp's
  // outstanding global stores
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// the copy lands in this CTA's shared memory; its bytes are counted on the barrier of the pair's
// leader (cluster address), which the MMA-issuing thread waits on for both CTAs' tiles
__device__ __forceinline__ void tmaLoad2dPair(void *dst, const CUtensorMap *map,
                                              uint32_t leader_bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
               " [%0], [%1, {%3, %4}], [%2];" ::"r"(smemAddr(dst)),
               "l"((uint64_t)map), "r"(leader_bar), "r"(x), "r"(y)
               : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tcCommitPair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
               " [%0], %1;" ::"r"(smemAddr(bar)),
               "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tcMmaPair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void tcFenceBefore() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcFenceAfter() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcCommit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smemAddr(bar))
               : "memory");
}
// D[tmem] (+)= A[smem descriptor] * B[smem descriptor]
__device__ __forceinline__ void tcMma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                      uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void tcLd8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                 "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tcLd32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
               "[%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                 "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
                 "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                 "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                 "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                 "=r"(v[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tcLd16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                 "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
                 "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tcSt16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
               "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
               "r"(v[15])
               : "memory");
}
__device__ __forceinline__ void tcWaitSt() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcWaitLd() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile whose rows are 64 bf16:
// 8-row groups are 1024 B apart (stride byte offset), layout type 2 = SWIZZLE_128B, descriptor
// version 1. Advancing by one 16-element K step adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t smemDesc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);      // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                      // descriptor version
  d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = 256 (the
// stacked hi and lo rows of the weight tile).
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) |
                            ((uint32_t)(TC_ACC_COLS >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
// the same for a CTA pair: M = 256, 128 rows in each CTA
constexpr uint32_t kIdescPair = (1u << 4) | (1u << 7) | (1u << 10) |
                                ((uint32_t)(TC_ACC_COLS >> 3) << 17) |
                                ((uint32_t)((2 * TC_M) >> 4) << 24);

// owner and row inside the owner's buffer of the 32-row group that starts at row `grow0` of the
// whole batch (a group never straddles two owners)
__device__ __forceinline__ void ownerOf(const TcKernelParams &p, int grow0, int &owner, int &lrow0) {
  if (p.owner_blk > 0) {
    const int blk = grow0 / p.owner_blk;
    owner = blk % p.n_owners;
    lrow0 = (blk / p.n_owners) * p.owner_blk + (grow0 - blk * p.owner_blk);
  } else {
    owner = grow0 / p.rows_per_owner;
    lrow0 = grow0 - owner * p.rows_per_owner;
  }
}

#define TC_TIMED_WAIT(acc, expr)                                                                   \
  ([&]() {                                                                                         \
    if (!timed) {                                                                                  \
      return (expr);                                                                               \
    }                                                                                              \
    const long long t_ = clock64();                                                                \
    const bool r_ = (expr);                                                                        \
    (acc) += clock64() - t_;                                                                       \
    return r_;                                                                                     \
  }())

// ---------------------------------------------------------------------------------------------
// the MVM kernel
// ---------------------------------------------------------------------------------------------
// PAIR = false: one CTA per work item (128 rows x one 128-column chunk).
// PAIR = true:  a cluster of two CTAs per work item of 256 rows; the MMAs are issued by the thread
//               of rank 0 for both CTAs (cta_group::2, M 256): each CTA's tensor core reads its own
//               128 rows of codes and half of the stacked weight tile from its own shared memory,
//               so the shared-memory traffic per SM and per FLOP drops by a third. Each CTA keeps
//               the accumulator rows of its own 128 rows in its own TMEM and runs its own epilogue.
// LINE: the std-dev of the output noise is read per output line from a table (out_noise_std > 0,
// single tile) and combined per element with the weight-noise term of the row.
template <bool BM, bool PAIR, bool CODES = false, bool LINE = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
    mvmTcKernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_bhi,
                const __grid_constant__ CUtensorMap tm_blo, const TcKernelParams p) {
  pdlEnter();
  constexpr int STAGES = PAIR ? TC2_STAGES : TC_STAGES;
  constexpr int STAGE_BYTES = PAIR ? TC2_STAGE_BYTES : TC_STAGE_BYTES;
  constexpr int KCH = PAIR ? TC2_KCH : TC_KCH;
  constexpr int CHUNK_BYTES = PAIR ? TC2_CHUNK_BYTES : TC_CHUNK_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = (uint64_t *)(smem + STAGES * STAGE_BYTES);
  uint64_t *full = bars;                    // [STAGES] operands landed in shared memory
  uint64_t *empty = bars + STAGES;          // [STAGES] MMAs have read the stage
  uint64_t *tmem_full = bars + 2 * STAGES;         // [TC_ACC_STAGES] accumulator complete
  uint64_t *tmem_empty = tmem_full + TC_ACC_STAGES; // [TC_ACC_STAGES] accumulator drained
  uint32_t *tmem_slot = (uint32_t *)(tmem_empty + TC_ACC_STAGES);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool timed = p.prof != nullptr;
  const int rank = PAIR ? (int)clusterCtaRank() : 0; // rank 0 of a pair issues the MMAs
  // persistent CTA (pair): work item w = (row block, 128-column chunk). Items are ordered so that
  // a group of `p.group` chunks is finished for every row block before the next group starts: the
  // group's weight operand (p.group * I * 256 KB) stays in L2 while the codes stream past once
  // per group.
  constexpr int ROWS = PAIR ? 2 * TC_M : TC_M; // rows per work item
  const int n_rb = (p.m + ROWS - 1) / ROWS;
  const int n_items = p.n_chunks * n_rb;
  const int worker = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x;
  const int n_workers = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x;
  auto item = [&](int w, int &chunk_idx, int &rb) {
    const int per_group = p.group * n_rb;
    const int g = w / per_group, rem = w - g * per_group;
    const int gsize = min(p.group, p.n_chunks - g * p.group); // last group may be smaller
    rb = rem / gsize;
    chunk_idx = g * p.group + (rem - rb * gsize);
    rb += p.rb_rotate;
    rb -= rb >= n_rb ? n_rb : 0;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbarInit(&full[s], 1);
      mbarInit(&empty[s], 1);
    }
    for (int b = 0; b < TC_ACC_STAGES; b++) {
      mbarInit(&tmem_full[b], 1);
      // the issuer waits for the epilogue warps of every CTA it computes for
      mbarInit(&tmem_empty[b], PAIR ? 2 * TC_EPI_WARPS : TC_EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TC_WARP_MMA) {
    // TMEM: all 512 columns = two accumulators of 128 lanes x (128 hi + 128 lo) fp32 columns.
    // For a pair the same warp of both CTAs allocates together, at the same shared-memory slot.
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smemAddr(tmem_slot)),
                   "r"(512)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smemAddr(tmem_slot)),
                   "r"(512)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (PAIR) {
    __syncwarp();
    clusterSync(); // the peer's barriers are initialised before anything arrives on them
  }
  tcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == TC_WARP_TMA) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int it = 0;
      int ps = 0;       // ring position and its phase parity
      uint32_t pph = 0;
      bool ok = true;
      long long w_empty = 0, w_issue = 0;
      for (int w = worker; w < n_items && ok; w += n_workers) {
      int chunk_idx, rb;
      item(w, chunk_idx, rb);
      const int r0 = rb * ROWS + rank * TC_M;
      for (int i = 0; i < p.I && ok; i++) {
        const int4 is = p.insplit[i];
        const int brow = i * p.nrows_pad + chunk_idx * TC_N;
        for (int kc0 = 0; kc0 < is.y; kc0 += KCH, it++) {
          const int nch = min(KCH, is.y - kc0); // chunks in this stage
          if (!TC_TIMED_WAIT(w_empty, mbarWait(&empty[ps], pph ^ 1u, abort_flag))) {
            atomicCAS(p.status, 0, TC_ERR_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const long long t_issue = timed ? clock64() : 0;
          if (PAIR) {
            // rank 0 announces the bytes of both CTAs on its barrier; both CTAs' copies count there
            const uint32_t leader_bar = mapaShared(smemAddr(&full[ps]), 0);
            if (rank == 0) {
              mbarExpectTx(&full[ps], 2 * nch * CHUNK_BYTES);
            }
#pragma unroll
            for (int c = 0; c < KCH; c++) {
              if (c < nch) {
                uint8_t *st = smem + ps * STAGE_BYTES + c * CHUNK_BYTES;
                const int kc = kc0 + c;
                tmaLoad2dPair(st, &tm_a, leader_bar, is.x + kc * TC_K, r0);
                tmaLoad2dPair(st + TC_STAGE_A, rank == 0 ? &tm_bhi : &tm_blo, leader_bar, kc * TC_K, brow);
              }
            }
          } else {
            mbarExpectTx(&full[ps], nch * CHUNK_BYTES);
#pragma unroll
            for (int c = 0; c < KCH; c++) {
              if (c < nch) {
                uint8_t *st = smem + ps * STAGE_BYTES + c * CHUNK_BYTES;
                const int kc = kc0 + c;
                tmaLoad2d(st, &tm_a, &full[ps], is.x + kc * TC_K, r0);
                tmaLoad2d(st + TC_STAGE_A, &tm_bhi, &full[ps], kc * TC_K, brow);
                tmaLoad2d(st + TC_STAGE_A + TC_STAGE_B, &tm_blo, &full[ps], kc * TC_K, brow);
              }
            }
          }
          if (++ps == STAGES) {
            ps = 0;
            pph ^= 1u;
          }
          if (timed) {
            w_issue += clock64() - t_issue;
          }
        }
      }
      }
      if (PAIR && ok) {
        // drain: the completions of the last MMAs arrive on this CTA's barriers from the thread
        // of rank 0 and must not find the CTA gone
        for (int k = it; k < it + STAGES; k++) {
          if (k >= STAGES && !mbarWait(&empty[k % STAGES], ((k / STAGES) & 1) ^ 1, abort_flag)) {
            break;
          }
        }
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 4] = w_empty;
        p.prof[blockIdx.x * 8 + 5] = w_issue;
      }
    }
  } else if (warp == TC_WARP_MMA) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && rank == 0) {
      int ai = 0;       // accumulator-buffer use counter
      int ms = 0;       // operand ring position and its phase parity
      uint32_t mph = 0;
      bool ok = true;
      long long w_full = 0, w_tmem = 0, w_mma = 0;
      const uint32_t smem0 = smemAddr(smem);
      const uint64_t desc_hi = smemDesc(0); // every field but the start address
      const long long t_start = clock64();
      for (int w = worker; w < n_items && ok; w += n_workers) {
      for (int i = 0; i < p.I && ok; i++, ai++) {
        const int nk = p.insplit[i].y;
        const int b = ai % TC_ACC_STAGES;
        if (!TC_TIMED_WAIT(w_tmem, mbarWait(&tmem_empty[b], ((ai / TC_ACC_STAGES) & 1) ^ 1, abort_flag))) {
          atomicCAS(p.status, 0, TC_ERR_TMEM_EMPTY);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tcFenceAfter();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * TC_ACC_COLS);
        for (int kc0 = 0; kc0 < nk; kc0 += KCH) {
          if (!TC_TIMED_WAIT(w_full, mbarWait(&full[ms], mph, abort_flag))) {
            atomicCAS(p.status, 0, TC_ERR_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tcFenceAfter();
          const long long t_mma = timed ? clock64() : 0;
          // descriptors differ between stages and chunks only in the start-address field
          // (16-byte units); +2 there = 32 bytes = 16 bf16 along K
          const uint32_t a0 = (smem0 + (uint32_t)(ms * STAGE_BYTES)) >> 4;
#pragma unroll
          for (int c = 0; c < KCH; c++) {
            if (c < nk - kc0) {
              // single CTA: the B descriptor starts at the hi tile and its 256 rows run on into
              // the lo tile. Pair: each CTA supplies 128 of the 256 B rows from the same offset.
              const uint64_t da = desc_hi | (uint64_t)(a0 + (uint32_t)(c * CHUNK_BYTES >> 4));
              const uint64_t db = da + (uint64_t)(TC_STAGE_A >> 4);
#pragma unroll
              for (int k = 0; k < TC_K / 16; k++) {
                const uint32_t accum = (kc0 > 0 || c > 0 || k > 0) ? 1u : 0u;
                if (PAIR) {
                  tcMmaPair(d_tmem, da + 2 * k, db + 2 * k, kIdescPair, accum);
                } else {
                  tcMma(d_tmem, da + 2 * k, db + 2 * k, kIdesc, accum);
                }
              }
            }
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (PAIR) {
            tcCommitPair(&empty[ms]);
          } else {
            tcCommit(&empty[ms]);
          }
          if (++ms == STAGES) {
            ms = 0;
            mph ^= 1u;
          }
          if (timed) {
            w_mma += clock64() - t_mma;
          }
        }
        if (ok) {
          // accumulator of in-split i is complete
          if (PAIR) {
            tcCommitPair(&tmem_full[b]);
          } else {
            tcCommit(&tmem_full[b]);
          }
        }
      }
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = w_full;
        p.prof[blockIdx.x * 8 + 1] = w_mma;
        p.prof[blockIdx.x * 8 + 2] = w_tmem;
        p.prof[blockIdx.x * 8 + 3] = clock64() - t_start;
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may access
    const int cbase = (warp >> 2) * TC_EPI_COLS; // first of this warp's columns
    const IOEff &io = p.io;
    const uint32_t tag = p.backward ? TAG_BWD_OUT : TAG_FWD_OUT;
    const bool adc = io.res_out > 0.0f;
    const float inv_res_out = adc ? 1.0f / io.res_out : 0.0f;
    const float kMagic = 12582912.0f; // 1.5 * 2^23: adding and subtracting rounds to nearest even
    const float in_codes = io.res_in * inv_res_out, bound_codes = io.out_bound * inv_res_out;
    // uniform over the launch: every row draws output noise and converts through the ADC
    const bool fast = adc && (io.out_noise > 0.0f ||
                              (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f));
    const Philox7Keys rkeys = philox7Keys(p.key);
    // eight accumulator columns of this thread's row: the product with hi + lo
    auto loadAcc8 = [](uint32_t ta, float (&acc)[8]) {
      uint32_t vh[8], vl[8];
      tcLd8(ta, vh);
      tcLd8(ta + (uint32_t)TC_N, vl);
      tcWaitLd();
#pragma unroll
      for (int j = 0; j < 8; j++) {
        acc[j] = __fadd_rn(__uint_as_float(vh[j]), __uint_as_float(vl[j]));
      }
    };
    bool ok = true;
    int ai = 0; // accumulator-buffer use counter, in step with the MMA issuer
    long long w_tfull = 0;
    const long long t_epi = clock64();
    for (int w = worker; w < n_items && ok; w += n_workers) {
    int chunk_idx, rb;
    item(w, chunk_idx, rb);
    const int4 ch = p.chunk[chunk_idx];
    const int row = rb * ROWS + rank * TC_M + q * 32 + lane;
    const bool row_ok = row < p.m;
    const uint32_t n4h = (uint32_t)((p.outn[ch.x] + 7) >> 3); // noise block pairs per row
    // first noise block pair of this warp's columns (chunks and column groups start on
    // multiples of 8 columns)
    const uint64_t ctr0 = (uint64_t)((ch.y + cbase) >> 3);
    bool exceeded = false;
    float sum[TC_EPI_COLS]; // running sums over the in-splits
#pragma unroll
    for (int c = 0; c < TC_EPI_COLS; c++) {
      sum[c] = 0.0f;
    }
    // per-row scalars of the next in-split are fetched one iteration ahead
    float sc_n = 0.0f, fac_n = 0.0f, vn_n = 0.0f;
    if (row_ok) {
      sc_n = p.scale[row];
      fac_n = p.factor[row];
      vn_n = p.vnorm[row];
      if (p.tile_scale) {
        fac_n *= p.tile_scale[ch.x];
      }
    }
    for (int i = 0; i < p.I; i++, ai++) {
      const int b = ai % TC_ACC_STAGES;
      const bool last = i + 1 == p.I;
      const float sc = sc_n, fac = fac_n;
      const float sigma = outputSigma(io, vn_n);
      // LINE: variance of the row's weight-noise term, to be joined with the line's own
      const float wv = (LINE && io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f)
                           ? io.w_noise * vn_n
                           : 0.0f;
      const float wv2 = wv * wv;
      auto lineSigma = [&](int col) -> float { // col: column within the chunk
        const float o = col < ch.w ? __ldg(p.onv + ch.z + col) : 0.0f;
        return wv2 > 0.0f ? sqrtf(fmaf(o, o, wv2)) : o;
      };
      if (row_ok && !last) {
        const long long si = (long long)(i + 1) * p.m + row;
        sc_n = p.scale[si];
        fac_n = p.factor[si];
        vn_n = p.vnorm[si];
        if (p.tile_scale) {
          fac_n *= p.tile_scale[(i + 1) * p.O + ch.x];
        }
      }
      const uint32_t tile_tag = tag + p.noise_id0 + (uint32_t)(i * p.noise_stride + ch.x);
      // the whole warp agrees on the outcome: what follows is warp-collective
      if (!__all_sync(0xffffffffu,
                      TC_TIMED_WAIT(w_tfull, mbarWait(&tmem_full[b], (ai / TC_ACC_STAGES) & 1, abort_flag)))) {
        atomicCAS(p.status, 0, TC_ERR_TMEM_FULL);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tcFenceAfter();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TC_ACC_COLS + cbase);
      const bool live = row_ok && sc != 0.0f;
      if (fast) {
        // Noisy regime with an ADC (the inference setting): the Gaussian decides the ADC code, so
        // the divisions of the exact chain become multiplications with the reciprocal step, all
        // in units of the ADC step. Straight-line code: rows without input (or beyond the batch)
        // run with factor 0, columns beyond the chunk are computed and never stored.
        const float sig_codes = live ? sigma * inv_res_out : 0.0f;
        const float fac_codes = live ? fac * io.res_out : 0.0f;
        const uint64_t ctr = ctr0 + (uint64_t)(p.row_base + row) * n4h;
        if (CODES) {
          // The rounded, clipped code stays in the low mantissa bits of (value + 1.5 * 2^23):
          // its low byte is the two's-complement code. Four codes per word, eight words per row.
          uint32_t cw[TC_EPI_COLS / 4];
          const float lo_m = kMagic - bound_codes, hi_m = kMagic + bound_codes;
#pragma unroll
          for (int c0 = 0; c0 < TC_EPI_COLS; c0 += 8) {
            float acc[8];
            loadAcc8(taddr + (uint32_t)c0, acc);
            float z[8];
            gauss8Keyed(rkeys, ctr + (uint64_t)(c0 >> 3), p.call, tile_tag, z);
            uint32_t bits[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
              float r = fmaf(z[j], sig_codes, acc[j] * in_codes) + kMagic;
              r = fminf(fmaxf(r, lo_m), hi_m);
              bits[j] = __float_as_uint(r);
            }
#pragma unroll
            for (int g = 0; g < 2; g++) {
              cw[(c0 >> 2) + g] =
                  __byte_perm(__byte_perm(bits[4 * g], bits[4 * g + 1], 0x0040),
                              __byte_perm(bits[4 * g + 2], bits[4 * g + 3], 0x0040), 0x5410);
            }
          }
          // this warp's 32 x 32 bytes are one contiguous 1 KB block at the owner: after an
          // exchange, every store instruction writes 512 contiguous bytes (rows 0-15, then 16-31)
          const int row0 = rb * ROWS + rank * TC_M + q * 32;
          if (row0 < p.m) {
            int owner, lrow0;
            ownerOf(p, p.row_base + row0, owner, lrow0);
            const long long n_total = p.out_ss; // columns of the whole layer
            const long long blk = (long long)(lrow0 >> 5) * (n_total >> 5) + ((ch.z + cbase) >> 5);
            uint8_t *dst = p.code_table[owner] + (long long)i * p.rows_per_owner * n_total + blk * 1024;
#pragma unroll
            for (int h = 0; h < 2; h++) {
              uint32_t v[4];
#pragma unroll
              for (int j = 0; j < TC_EPI_COLS / 4; j++) {
                const uint32_t t = __shfl_sync(0xffffffffu, cw[j], (lane >> 1) + 16 * h);
                if ((j >> 2) == (lane & 1)) {
                  v[j & 3] = t;
                }
              }
              *reinterpret_cast<uint4 *>(dst + h * 512 + lane * 16) = make_uint4(v[0], v[1], v[2], v[3]);
            }
            if (ch.z == 0 && cbase == 0 && row_ok) {
              p.fac_table[owner][(long long)i * p.rows_per_owner + lrow0 + (row - row0)] = fac_codes;
            }
          }
        } else {
#pragma unroll
        for (int c0 = 0; c0 < TC_EPI_COLS; c0 += 8) {
          float acc[8];
          loadAcc8(taddr + (uint32_t)c0, acc);
          float z[8];
          gauss8Keyed(rkeys, ctr + (uint64_t)(c0 >> 3), p.call, tile_tag, z);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float sg = LINE ? (live ? lineSigma(cbase + c0 + j) * inv_res_out : 0.0f) : sig_codes;
            float r = fmaf(z[j], sg, acc[j] * in_codes);
            r = (r + kMagic) - kMagic; // round to nearest even
            if (BM && cbase + c0 + j < ch.w) {
              exceeded = exceeded || (r > bound_codes) || (io.bm_test_negative_bound && r < -bound_codes);
            }
            r = fminf(fmaxf(r, -bound_codes), bound_codes);
            sum[c0 + j] = fmaf(r, fac_codes, sum[c0 + j]);
          }
        }
        }
      } else {
#pragma unroll
        for (int c0 = 0; c0 < TC_EPI_COLS; c0 += 8) {
          float acc[8];
          loadAcc8(taddr + (uint32_t)c0, acc);
          if (live) {
            float z[8];
            if (sigma > 0.0f && cbase + c0 < ch.w) {
              gauss8Keyed(rkeys, ctr0 + (uint64_t)(p.row_base + row) * n4h + (uint64_t)(c0 >> 3), p.call,
                          tile_tag, z);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
              if (cbase + c0 + j < ch.w) {
                float y;
                if (sigma > 0.0f) { // noise without an ADC
                  y = fmaf(acc[j], io.res_in, (LINE ? lineSigma(cbase + c0 + j) : sigma) * z[j]);
                  if (BM) {
                    exceeded = exceeded || (y > io.out_bound) ||
                               (io.bm_test_negative_bound && y < -io.out_bound);
                  }
                  y = fminf(fmaxf(y, -io.out_bound), io.out_bound);
                } else {
                  // exact chain: the MMA summed integer codes times weights; one multiply by
                  // the DAC step gives sum(v * w)
                  y = finalizeOutput(io, __fmul_rn(acc[j], io.res_in), 0.0f, 0.0f, exceeded);
                }
                sum[c0 + j] = fmaf(y, fac, sum[c0 + j]);
              }
            }
          }
        }
      }
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) {
          // the issuer's "accumulator drained" barriers live in rank 0 of the pair
          mbarArriveCluster(mapaShared(smemAddr(&tmem_empty[b]), 0));
        } else {
          mbarArrive(&tmem_empty[b]);
        }
      }
    }
    if (ok && row_ok && exceeded && io.bm != AB200_BM_NONE && p.flags != nullptr) {
      atomicOr(&p.flags[row], 1);
    }
    if (CODES) {
      // everything went out in-split by in-split
    } else if (ok && (p.out_table || p.row_stores)) {
      // Scatter to the row-block owners, possibly peer memory: transpose the warp's 32 x 32
      // block in registers (five exchange steps) so that every store instruction writes 128
      // contiguous bytes of one row - over NVLink the 16-byte pieces of the row-per-lane layout
      // would each travel alone.
#pragma unroll
      for (int st = 16; st >= 1; st >>= 1) {
#pragma unroll
        for (int c = 0; c < TC_EPI_COLS; c++) {
          if ((c & st) == 0) {
            const bool upper = (lane & st) != 0;
            const float send = upper ? sum[c] : sum[c | st];
            const float recv = __shfl_xor_sync(0xffffffffu, send, st);
            if (upper) {
              sum[c] = recv;
            } else {
              sum[c | st] = recv;
            }
          }
        }
      }
      // now sum[r] = element (row r of this warp's row group, column cbase + lane)
      const int col = cbase + lane;
      const int row0 = rb * ROWS + rank * TC_M + q * 32;
      if (col < ch.w && row0 < p.m) {
        const float b = p.bias ? p.bias[ch.z + col] : 0.0f;
        float *o;
        if (p.out_table) {
          int owner, lrow0;
          ownerOf(p, p.row_base + row0, owner, lrow0);
          o = p.out_table[owner] + (long long)lrow0 * p.out_ss + ch.z + col;
        } else {
          o = p.out + (long long)row0 * p.out_ss + ch.z + col;
        }
#pragma unroll
        for (int r = 0; r < 32; r++) {
          if (row0 + r < p.m) {
            o[(long long)r * p.out_ss] = sum[r] + b;
          }
        }
      }
    } else if (ok && row_ok && p.out_t_rows > 0) {
      const int grow = p.row_base + row; // row of the whole batch
      const int blk = grow / p.out_t_rows, l = grow - blk * p.out_t_rows;
      float *o = p.out + ((long long)blk * p.out_ss + ch.z + cbase) * p.out_t_rows + l;
#pragma unroll
      for (int c = 0; c < TC_EPI_COLS; c++) {
        if (cbase + c < ch.w) {
          o[(long long)c * p.out_t_rows] = sum[c] + (p.bias ? p.bias[ch.z + cbase + c] : 0.0f);
        }
      }
    } else if (ok && row_ok) {
      const bool vec = ((p.out_ss & 3) == 0) && ((ch.z & 3) == 0) &&
                       ((((uintptr_t)p.out) & 15) == 0) && !p.accumulate;
      float *orow = p.out + (long long)row * p.out_ss + ch.z + cbase;
      if (p.bias) {
#pragma unroll
        for (int c = 0; c < TC_EPI_COLS; c++) {
          if (cbase + c < ch.w) {
            sum[c] += p.bias[ch.z + cbase + c];
          }
        }
      }
#pragma unroll
      for (int c = 0; c < TC_EPI_COLS; c += 4) {
        const int cl = cbase + c;
        if (vec && cl + 3 < ch.w) {
          *reinterpret_cast<float4 *>(orow + c) =
              make_float4(sum[c], sum[c + 1], sum[c + 2], sum[c + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            if (cl + j < ch.w) {
              float *o = orow + c + j;
              *o = p.accumulate ? *o + sum[c + j] : sum[c + j];
            }
          }
        }
      }
    }
    }
    if (p.prof && threadIdx.x == 0) {
      p.prof[blockIdx.x * 8 + 6] = w_tfull;
      p.prof[blockIdx.x * 8 + 7] = clock64() - t_epi;
    }
  }

  // teardown: everyone meets here, also after a time-out
  if (p.flag_table != nullptr) {
    __threadfence_system(); // this thread's stores, peer memory included, before the signal
  }
  tcFenceBefore();
  __syncthreads();
  if (p.flag_table != nullptr && threadIdx.x == 0 && *abort_flag == 0) {
    __threadfence();
    const int finished = atomicAdd(p.done_ctr, 1);
    if (finished == (int)gridDim.x - 1) {
      // every CTA of this launch has passed its fence: tell the owners
      atomicExch(p.done_ctr, 0);
      __threadfence_system();
      for (int q = 0; q < p.n_owners; q++) {
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flag_table[q]), "r"(p.epoch) : "memory");
      }
    }
  }
  if (*abort_flag != 0 && threadIdx.x == 0) {
    // give copies that are still in flight time to land before the shared memory is released
    const long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 2000000ull) {
      __nanosleep(1000);
    }
  }
  __syncthreads();
  if (PAIR) {
    // neither CTA leaves while its peer may still arrive on its barriers or feed its tensor core
    __syncwarp();
    clusterSync();
  }
  if (warp == TC_WARP_MMA) {
    tcFenceAfter();
    if (PAIR) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                   : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                   : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------------------
// DAC: one warp per (row, in-split)
// ---------------------------------------------------------------------------------------------
struct DacParams {
  const float *in;
  long long in_ss;
  int m, I, kpad;
  const int4 *insplit; // {k0, n_k_stages, K_i, in_off}
  __nv_bfloat16 *codes;
  long long codes_ld;
  float *scale, *factor, *vnorm, *sval;
  int *flags;
  IOEff io;
  float alpha;
  int backward;
  float code_bound; // largest |code| = inp_bound / res_in
  float inv_res_in; // 1 / res_in: first guess of the DAC code
  // rows gathered from whole images at `in` (null index: plain rows); row 0 of this launch is
  // row g_row0 of the gathered batch
  RowGather gather;
  int g_row0;
};

// rint((x * scale) / res_in), clipped: the reference's DAC in its own association. The division is
// only carried out where a product with the reciprocal step lands within 1e-4 of a half-integer
// (only there can the two round to different codes: the product is off by at most 2e-5 at the
// largest code, the correctly rounded quotient by 4e-6); elsewhere both give the same integer.
__device__ __forceinline__ float dacCode(const DacParams &p, float x, float scale) {
  const float v = __fmul_rn(x, scale);
  const float q = __fmul_rn(v, p.inv_res_in);
  float code = rintf(q);
  if (fabsf(__fsub_rn(q, code)) > 0.4999f) {
    code = rintf(__fdiv_rn(v, p.io.res_in));
  }
  return fminf(fmaxf(code, -p.code_bound), p.code_bound);
}
__device__ __forceinline__ void dacRowScalars(const DacParams &p, int i, int row, float sval, float scale,
                                              float sumsq) {
  const long long si = (long long)i * p.m + row;
  p.scale[si] = scale;
  p.factor[si] = outputFactor(p.io, p.alpha, sval, scale, p.backward);
  p.vnorm[si] = sqrtf(sumsq) * p.io.res_in;
  if (p.sval) {
    p.sval[si] = sval;
  }
  if (p.flags) {
    p.flags[si] = 0;
  }
}

// any in-split length and alignment: one warp per (row, in-split), two passes over the row (the
// second one hits L1 / L2)
__global__ void __launch_bounds__(256) dacQuantizeKernel(DacParams p) {
  pdlEnter();
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)p.m * p.I) {
    return;
  }
  const int i = (int)(w / p.m), row = (int)(w % p.m);
  const int4 is = p.insplit[i];
  const int K = is.z;
  const float *x = p.in + (long long)row * p.in_ss + is.w;
  const IOEff &io = p.io;
  float amax = 0.0f;
  if (io.nm == AB200_NM_ABS_MAX) {
#pragma unroll 8
    for (int k = lane; k < K; k += 32) {
      amax = fmaxf(amax, fabsf(x[k]));
    }
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
  }
  const float sval = nmValue(io, amax);
  const float scale = inputScale(io, sval, 1.0f, !p.backward);
  __nv_bfloat16 *c = p.codes + (long long)row * p.codes_ld + is.x;
  float acc = 0.0f;
#pragma unroll 4
  for (int k = lane; k < p.kpad; k += 32) {
    float code = 0.0f;
    if (k < K && scale != 0.0f) {
      code = dacCode(p, x[k], scale);
    }
    c[k] = __float2bfloat16_rn(code);
    acc = fmaf(code, code, acc);
  }
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
  }
  if (lane == 0) {
    dacRowScalars(p, i, row, sval, scale, acc);
  }
}

// In-splits of at most 512 inputs whose rows start on 16-byte boundaries: one warp per row; an
// in-split sits in the registers of the warp (four float4 per lane) and is read once. In-splits go
// through in pairs: their reductions across the warp are independent chains of shuffles, which
// overlap.
struct DacRegs {
  float4 v[4];
};
__device__ __forceinline__ void dacLoadRow(const DacParams &p, int i, int row, int lane, DacRegs &r) {
  const int4 is = p.insplit[i];
  const float4 *x = reinterpret_cast<const float4 *>(p.in + (long long)row * p.in_ss + is.w);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int k = 4 * (lane + 32 * j);
    r.v[j] = k < is.z ? __ldg(x + lane + 32 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
template <int NI>
__device__ __forceinline__ void dacQuantRows(const DacParams &p, int i0, int row, int lane,
                                             const DacRegs (&r)[NI]) {
  const IOEff &io = p.io;
  float amax[NI];
#pragma unroll
  for (int n = 0; n < NI; n++) {
    amax[n] = 0.0f;
    if (io.nm == AB200_NM_ABS_MAX) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        amax[n] = fmaxf(fmaxf(amax[n], fmaxf(fabsf(r[n].v[j].x), fabsf(r[n].v[j].y))),
                        fmaxf(fabsf(r[n].v[j].z), fabsf(r[n].v[j].w)));
      }
    }
  }
  if (io.nm == AB200_NM_ABS_MAX) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int n = 0; n < NI; n++) {
        amax[n] = fmaxf(amax[n], __shfl_xor_sync(0xffffffffu, amax[n], o));
      }
    }
  }
  float sval[NI], scale[NI], acc[NI];
#pragma unroll
  for (int n = 0; n < NI; n++) {
    const int4 is = p.insplit[i0 + n];
    sval[n] = nmValue(io, amax[n]);
    scale[n] = inputScale(io, sval[n], 1.0f, !p.backward);
    __nv_bfloat16 *c = p.codes + (long long)row * p.codes_ld + is.x;
    acc[n] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = 4 * (lane + 32 * j);
      if (k < p.kpad) {
        float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
        if (k < is.z && scale[n] != 0.0f) {
          c0 = dacCode(p, r[n].v[j].x, scale[n]);
          c1 = dacCode(p, r[n].v[j].y, scale[n]);
          c2 = dacCode(p, r[n].v[j].z, scale[n]);
          c3 = dacCode(p, r[n].v[j].w, scale[n]);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(c0, c1), hi = __floats2bfloat162_rn(c2, c3);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t *>(&lo);
        pk.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(c + k) = pk;
        acc[n] = fmaf(c0, c0, acc[n]);
        acc[n] = fmaf(c1, c1, acc[n]);
        acc[n] = fmaf(c2, c2, acc[n]);
        acc[n] = fmaf(c3, c3, acc[n]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int n = 0; n < NI; n++) {
      acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], o);
    }
  }
#pragma unroll
  for (int n = 0; n < NI; n++) {
    if (lane == n) {
      dacRowScalars(p, i0 + n, row, sval[n], scale[n], acc[n]);
    }
  }
}
// Small CTAs with at most 64 registers per thread: one of them fits on an SM beside a CTA of the
// MMA kernel, several when the kernel runs alone.
__global__ void __launch_bounds__(128, 8) dacQuantizeRowKernel(DacParams p) {
  pdlEnter();
  const int row = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= p.m) {
    return;
  }
  for (int i = 0; i < p.I; i += 2) {
    if (i + 1 < p.I) {
      DacRegs r[2];
      dacLoadRow(p, i, row, lane, r[0]);
      dacLoadRow(p, i + 1, row, lane, r[1]);
      dacQuantRows<2>(p, i, row, lane, r);
    } else {
      DacRegs r[1];
      dacLoadRow(p, i, row, lane, r[0]);
      dacQuantRows<1>(p, i, row, lane, r);
    }
  }
}

// In-splits longer than 512 inputs (a tile that is not mapped, e.g. the 2304 inputs of a 3 x 3
// convolution over 256 channels) with 16-byte aligned rows: one warp per (row, in-split), float4
// loads, two passes over the row - the second one finds it in L1 / L2.
__global__ void __launch_bounds__(256) dacQuantizeLongRowKernel(DacParams p) {
  pdlEnter();
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)p.m * p.I) {
    return;
  }
  const int i = (int)(wid / p.m), row = (int)(wid % p.m);
  const int4 is = p.insplit[i];
  const int K4 = is.z >> 2;
  const float4 *x = reinterpret_cast<const float4 *>(p.in + (long long)row * p.in_ss + is.w);
  const IOEff &io = p.io;
  float amax = 0.0f;
  if (io.nm == AB200_NM_ABS_MAX) {
    float a0 = 0.0f, a1 = 0.0f;
    int k = lane;
    for (; k + 32 < K4; k += 64) {
      const float4 u = __ldg(x + k), v = __ldg(x + k + 32);
      a0 = fmaxf(fmaxf(a0, fmaxf(fabsf(u.x), fabsf(u.y))), fmaxf(fabsf(u.z), fabsf(u.w)));
      a1 = fmaxf(fmaxf(a1, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
    if (k < K4) {
      const float4 u = __ldg(x + k);
      a0 = fmaxf(fmaxf(a0, fmaxf(fabsf(u.x), fabsf(u.y))), fmaxf(fabsf(u.z), fabsf(u.w)));
    }
    amax = fmaxf(a0, a1);
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
  }
  const float sval = nmValue(io, amax);
  const float scale = inputScale(io, sval, 1.0f, !p.backward);
  __nv_bfloat16 *c = p.codes + (long long)row * p.codes_ld + is.x;
  float acc = 0.0f;
  const int KP4 = p.kpad >> 2;
#pragma unroll 2
  for (int k = lane; k < KP4; k += 32) {
    float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
    if (k < K4 && scale != 0.0f) {
      const float4 v = __ldg(x + k);
      c0 = dacCode(p, v.x, scale);
      c1 = dacCode(p, v.y, scale);
      c2 = dacCode(p, v.z, scale);
      c3 = dacCode(p, v.w, scale);
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(c0, c1), hi = __floats2bfloat162_rn(c2, c3);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t *>(&lo);
    pk.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(c + 4 * k) = pk;
    acc = fmaf(c0, c0, acc);
    acc = fmaf(c1, c1, acc);
    acc = fmaf(c2, c2, acc);
    acc = fmaf(c3, c3, acc);
  }
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
  }
  if (lane == 0) {
    dacRowScalars(p, i, row, sval, scale, acc);
  }
}

// Rows gathered from whole images through the index array of the indexed convolution interface:
// one warp per (row, in-split). The gathered values are staged in the warp's slice of shared
// memory between the abs-max pass and the quantisation, so every index and image element is read
// once and the sample-major matrix of the unfolded images never exists in HBM.
constexpr int kGatherWarps = 4;
__global__ void __launch_bounds__(kGatherWarps * 32) dacQuantizeGatherKernel(DacParams p) {
  pdlEnter();
  extern __shared__ __align__(16) float g_sh[]; // [kGatherWarps][kpad]
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)p.m * p.I) {
    return;
  }
  const int i = (int)(wid / p.m), row = (int)(wid % p.m);
  const int4 is = p.insplit[i];
  const int K = is.z;
  const int grow = p.g_row0 + row;
  const int n = grow / p.gather.m_batch, l = grow - n * p.gather.m_batch;
  const int32_t *ix = p.gather.idx + (long long)l * p.gather.ld + is.w;
  const float *img = p.in + (long long)n * p.gather.image_size;
  float *sh = g_sh + (threadIdx.x >> 5) * p.kpad;
  const IOEff &io = p.io;
  float amax = 0.0f;
  // sixteen index loads, then sixteen image loads in flight per lane: the two dependent loads of
  // an element are latency, not bandwidth
  constexpr int kU = 16;
  for (int k0 = lane; k0 < p.kpad; k0 += 32 * kU) {
    int j[kU];
#pragma unroll
    for (int u = 0; u < kU; u++) {
      const int k = k0 + 32 * u;
      j[u] = k < K ? __ldg(ix + k) : 0;
    }
    float v[kU];
#pragma unroll
    for (int u = 0; u < kU; u++) {
      v[u] = j[u] <= 1 ? (float)j[u] : __ldg(img + (j[u] - 2));
    }
#pragma unroll
    for (int u = 0; u < kU; u++) {
      const int k = k0 + 32 * u;
      if (k < p.kpad) {
        sh[k] = v[u];
      }
      amax = fmaxf(amax, fabsf(v[u]));
    }
  }
  if (io.nm == AB200_NM_ABS_MAX) {
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
  } else {
    amax = 0.0f;
  }
  __syncwarp();
  const float sval = nmValue(io, amax);
  const float scale = inputScale(io, sval, 1.0f, !p.backward);
  __nv_bfloat16 *c = p.codes + (long long)row * p.codes_ld + is.x;
  float acc = 0.0f;
  const int KP4 = p.kpad >> 2;
  const float4 *sh4 = reinterpret_cast<const float4 *>(sh);
#pragma unroll 2
  for (int k = lane; k < KP4; k += 32) {
    float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
    if (scale != 0.0f) {
      const float4 v = sh4[k]; // zero beyond K: code 0
      c0 = dacCode(p, v.x, scale);
      c1 = dacCode(p, v.y, scale);
      c2 = dacCode(p, v.z, scale);
      c3 = dacCode(p, v.w, scale);
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(c0, c1), hi = __floats2bfloat162_rn(c2, c3);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t *>(&lo);
    pk.y = *reinterpret_cast<const uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(c + 4 * k) = pk;
    acc = fmaf(c0, c0, acc);
    acc = fmaf(c1, c1, acc);
    acc = fmaf(c2, c2, acc);
    acc = fmaf(c3, c3, acc);
  }
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
  }
  if (lane == 0) {
    dacRowScalars(p, i, row, sval, scale, acc);
  }
}

// B[n][k] = w[k * wk + n * wn]  ->  bf16 hi, lo at row (row0 + n) of the padded operand
__global__ void __launch_bounds__(256)
    splitWeightsKernel(const float *w, long long wk, long long wn, int N, int K, __nv_bfloat16 *hi,
                       __nv_bfloat16 *lo, long long row0, int kpad) {
  pdlEnter();
  __shared__ float t[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32; // bx along k, by along n
  const bool k_fast = wk == 1;                          // which index is contiguous in memory
  for (int r = threadIdx.y; r < 32; r += 8) {
    // read with the contiguous index across threadIdx.x
    int k = k_fast ? bx + threadIdx.x : bx + r;
    int n = k_fast ? by + r : by + threadIdx.x;
    float v = (k < K && n < N) ? w[(long long)k * wk + (long long)n * wn] : 0.0f;
    if (k_fast) {
      t[r][threadIdx.x] = v; // t[n][k]
    } else {
      t[threadIdx.x][r] = v; // t[n][k]
    }
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8) {
    int n = by + r, k = bx + threadIdx.x;
    if (n < N && k < K) {
      float v = t[r][threadIdx.x];
      __nv_bfloat16 h = __float2bfloat16_rn(v);
      float rem = v - __bfloat162float(h);
      long long o = (row0 + n) * (long long)kpad + k;
      hi[o] = h;
      lo[o] = __float2bfloat16_rn(rem);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res);
    if (e == cudaSuccess && res == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  if (!fn) {
    AB200_FATAL("cuTensorMapEncodeTiled is not available from the CUDA driver");
  }
  return fn;
}

// 2-D bf16 tensor [rows][cols] with row pitch `ld` elements; box = 64 columns x 128 rows,
// 128-byte swizzle, out-of-range elements read as zero.
static CUtensorMap makeMap(void *base, uint64_t rows, uint64_t cols, uint64_t ld) {
  CUtensorMap map;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TC_K, (cuuint32_t)TC_M};
  cuuint32_t estr[2] = {1, 1};
  if (((uintptr_t)base & 15) != 0 || (strides[0] & 15) != 0) {
    AB200_FATAL("tensor map: base and row pitch must be 16-byte aligned");
  }
  CUresult r = encodeTiled()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box,
                             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    AB200_FATAL("cuTensorMapEncodeTiled failed with code " << (int)r);
  }
  return map;
}

// The scatter of ADC codes needs the noisy regime with an ADC whose codes fit a signed byte, and
// no bound management (nothing is re-run after the codes have left).
bool TcEngine::codesSupported(const IOEff &io) {
  if (!ioSupported(io) || io.bm != AB200_BM_NONE || !(io.res_out > 0.0f)) {
    return false;
  }
  const bool noisy = io.out_noise > 0.0f ||
                     (io.w_noise_type == AB200_WNOISE_ADDITIVE_CONSTANT && io.w_noise > 0.0f);
  const float bc = io.out_bound / io.res_out;
  return noisy && bc <= 127.0f && fabsf(bc - rintf(bc)) < 1e-3f;
}

bool TcEngine::gatherSupported(int in_size) {
  // kGatherWarps rows of the padded width, fp32, in the shared memory of one CTA
  const size_t kpad = ((size_t)in_size + 63) / 64 * 64;
  return kGatherWarps * kpad * sizeof(float) <= 200 * 1024;
}

bool TcEngine::ioSupported(const IOEff &io, bool line_table) {
  if (io.is_perfect || !(io.res_in > 0.0f) || !(io.inp_bound < 1e30f)) {
    return false;
  }
  // input noise takes the DAC output off the integer grid; asymmetries and stochastic rounding
  // are left to the CUDA-core kernels too
  if (io.inp_noise > 0.0f || io.inp_asym != 1.0f || io.out_asym != 1.0f || io.inp_sto_round ||
      io.out_sto_round) {
    return false;
  }
  // a noise std-dev per output line or per element (PCMRead) likewise, and the non-idealities
  // of the output lines (IR drop, voltage offsets, series resistance, non-linearity)
  if ((io.w_noise_type == AB200_WNOISE_PCM_READ && io.w_noise > 0.0f) || ioNeedsLineChain(io)) {
    return false;
  }
  // a std-dev of the output noise per line: only where the caller hands over its table
  if (io.out_noise_std > 0.0f && !line_table) {
    return false;
  }
  // the DAC kernel of this path knows the common noise-management types only, and the re-run
  // kernel of IterativeWorstCase changes the noise-management value per row
  if ((io.nm != AB200_NM_NONE && io.nm != AB200_NM_ABS_MAX && io.nm != AB200_NM_CONSTANT) ||
      io.bm == AB200_BM_ITERATIVE_WORST_CASE) {
    return false;
  }
  float cb = io.inp_bound / io.res_in;
  float r = rintf(cb);
  return r >= 1.0f && r <= 256.0f && fabsf(cb - r) < 1e-3f;
}

TcEngine::TcEngine(int device) : device_(device) {
  AB200_CUDA(cudaSetDevice(device_));
  AB200_CUDA(cudaHostAlloc(&status_host_, sizeof(int), cudaHostAllocMapped));
  *status_host_ = 0;
  AB200_CUDA(cudaHostGetDevicePointer(&status_dev_, status_host_, 0));
}

TcEngine::~TcEngine() {
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaFree(op_hi_);
  cudaFree(op_lo_);
  cudaFree(codes_);
  cudaFree(scale_);
  cudaFree(factor_);
  cudaFree(vnorm_);
  cudaFree(sval_);
  cudaFree(flags_);
  cudaFree(chunk_tab_);
  cudaFree(insplit_tab_);
  cudaFree(outn_tab_);
  cudaFree(done_ctr_);
  if (side_) {
    cudaStreamDestroy(side_);
    cudaEventDestroy(ev_fork_);
    cudaEventDestroy(ev_join_);
  }
  cudaFreeHost(status_host_);
  if (prev >= 0) {
    cudaSetDevice(prev);
  }
}

void TcEngine::checkStatus() {
  if (status_host_ && *status_host_ != 0) {
    int code = *status_host_;
    *status_host_ = 0;
    AB200_FATAL("tensor-core MVM kernel gave up on a bounded wait (status " << code << ")");
  }
}

void TcEngine::configure(const std::vector<int> &in_sizes, const std::vector<int> &out_sizes) {
  AB200_CUDA(cudaSetDevice(device_));
  in_sizes_ = in_sizes;
  out_sizes_ = out_sizes;
  int kmax = 0;
  for (int k : in_sizes) {
    kmax = std::max(kmax, k);
  }
  kpad_ = (kmax + TC_K - 1) / TC_K * TC_K;
  std::vector<int4> chunks;
  out_off_.clear();
  int off = 0;
  for (int o = 0; o < (int)out_sizes.size(); o++) {
    out_off_.push_back(off);
    for (int c = 0; c < out_sizes[o]; c += TC_N) {
      chunks.push_back(make_int4(o, c, off + c, std::min(TC_N, out_sizes[o] - c)));
    }
    off += out_sizes[o];
  }
  n_chunks_ = (int)chunks.size();
  nrows_pad_ = n_chunks_ * TC_N;
  in_off_.clear();
  std::vector<int4> ins;
  off = 0;
  for (int i = 0; i < (int)in_sizes.size(); i++) {
    in_off_.push_back(off);
    ins.push_back(make_int4(i * kpad_, (in_sizes[i] + TC_K - 1) / TC_K, in_sizes[i], off));
    off += in_sizes[i];
  }
  const size_t op_elems = (size_t)in_sizes.size() * nrows_pad_ * kpad_;
  cudaFree(op_hi_);
  cudaFree(op_lo_);
  cudaFree(chunk_tab_);
  cudaFree(insplit_tab_);
  cudaFree(outn_tab_);
  AB200_CUDA(cudaMalloc(&op_hi_, op_elems * 2));
  AB200_CUDA(cudaMalloc(&op_lo_, op_elems * 2));
  AB200_CUDA(cudaMemset(op_hi_, 0, op_elems * 2));
  AB200_CUDA(cudaMemset(op_lo_, 0, op_elems * 2));
  AB200_CUDA(cudaMalloc(&chunk_tab_, chunks.size() * sizeof(int4)));
  AB200_CUDA(cudaMemcpy(chunk_tab_, chunks.data(), chunks.size() * sizeof(int4), cudaMemcpyHostToDevice));
  AB200_CUDA(cudaMalloc(&insplit_tab_, ins.size() * sizeof(int4)));
  AB200_CUDA(cudaMemcpy(insplit_tab_, ins.data(), ins.size() * sizeof(int4), cudaMemcpyHostToDevice));
  AB200_CUDA(cudaMalloc(&outn_tab_, out_sizes.size() * sizeof(int)));
  AB200_CUDA(cudaMemcpy(outn_tab_, out_sizes.data(), out_sizes.size() * sizeof(int), cudaMemcpyHostToDevice));
  m_cap_ = 0;
}

void TcEngine::loadOperand(int i, int o, const float *w, long long wk, long long wn,
                           cudaStream_t s) {
  AB200_CUDA(cudaSetDevice(device_));
  const int N = out_sizes_[o], K = in_sizes_[i];
  // row of the padded operand where out-split o starts: its first chunk * 128
  long long chunk0 = 0;
  for (int oo = 0; oo < o; oo++) {
    chunk0 += (out_sizes_[oo] + TC_N - 1) / TC_N;
  }
  const long long row0 = (long long)i * nrows_pad_ + chunk0 * TC_N;
  dim3 grid((K + 31) / 32, (N + 31) / 32), block(32, 8);
  AB200_CUDA(launchChained(splitWeightsKernel, grid, block, 0, s, w, wk, wn, N, K, (__nv_bfloat16 *)op_hi_,
                           (__nv_bfloat16 *)op_lo_, row0, kpad_));
  AB200_LAUNCH_CHECK();
}

void TcEngine::ensureBatch(int m) {
  if (m <= m_cap_) {
    return;
  }
  AB200_CUDA(cudaDeviceSynchronize());
  cudaFree(codes_);
  cudaFree(scale_);
  cudaFree(factor_);
  cudaFree(vnorm_);
  cudaFree(sval_);
  cudaFree(flags_);
  const int cap = m + m / 4 + 128;
  const size_t I = in_sizes_.size();
  AB200_CUDA(cudaMalloc(&codes_, (size_t)cap * I * kpad_ * 2));
  AB200_CUDA(cudaMalloc(&scale_, (size_t)cap * I * sizeof(float)));
  AB200_CUDA(cudaMalloc(&factor_, (size_t)cap * I * sizeof(float)));
  AB200_CUDA(cudaMalloc(&vnorm_, (size_t)cap * I * sizeof(float)));
  AB200_CUDA(cudaMalloc(&sval_, (size_t)cap * I * sizeof(float)));
  AB200_CUDA(cudaMalloc(&flags_, (size_t)cap * I * sizeof(int)));
  m_cap_ = cap;
}

// CTA pairs whenever there are at least two 128-row blocks (and the mode allows it)
static bool usePairs(int m) { return mvmPath() != 3 && m > TC_M; }
// diagnostics: AB200_TC_SPLIT=1 cuts large batches into two halves (see TcEngine::run)
static bool mvmSplit() {
  static const bool on = [] {
    const char *e = getenv("AB200_TC_SPLIT");
    return e && e[0] == '1';
  }();
  return on;
}
static int pair_rows(int m) { return usePairs(m) ? 2 * TC_M : TC_M; }

void TcEngine::run(const Run &r, cudaStream_t s) {
  AB200_CUDA(cudaSetDevice(device_));
  checkStatus();
  if (r.m <= 0) {
    return;
  }
  const int I = (int)in_sizes_.size();
  if (!ioSupported(r.io, r.onv != nullptr)) {
    AB200_FATAL("tensor-core MVM: IO settings not expressible as integer DAC codes");
  }
  ensureBatch(r.m);
  if (r.scale != nullptr && I != 1) {
    AB200_FATAL("tensor-core MVM: caller-owned scratch needs a single in-split");
  }
  // Two launches per batch half when the batch is large: the DAC kernel of the second half runs
  // on a side stream beside the MMA kernel of the first (which leaves registers and threads for
  // one such CTA per SM), so only the first half's DAC is exposed. Each half keeps several waves
  // of work items. Runs that scatter to row-block owners stay whole (their sweep order is part of
  // the protocol between the ranks).
  const int rows_item = pair_rows(r.m);
  int n_sm = 0;
  AB200_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device_));
  const int workers = usePairs(r.m) ? n_sm / 2 : n_sm;
  const int half_blocks = (r.m / rows_item) / 2;
  const bool split = mvmSplit() && r.out_table == nullptr && r.code_table == nullptr && half_blocks > 0 &&
                     (long long)half_blocks * n_chunks_ >= 4LL * workers;
  if (!split) {
    launchDac(r, 0, r.m, s);
    launchMma(r, 0, r.m, s);
    return;
  }
  if (!side_) {
    AB200_CUDA(cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking));
    AB200_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
    AB200_CUDA(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming));
  }
  const int rows_a = half_blocks * rows_item;
  launchDac(r, 0, rows_a, s);
  AB200_CUDA(cudaEventRecord(ev_fork_, s)); // the side stream starts after the first half's DAC
  AB200_CUDA(cudaStreamWaitEvent(side_, ev_fork_, 0));
  launchDac(r, rows_a, r.m - rows_a, side_);
  AB200_CUDA(cudaEventRecord(ev_join_, side_));
  launchMma(r, 0, rows_a, s);
  AB200_CUDA(cudaStreamWaitEvent(s, ev_join_, 0));
  launchMma(r, rows_a, r.m - rows_a, s);
}

// per-row scratch of the rows [row0, row0 + rows): the caller's arrays (single in-split, indexed
// by row) or a slice of the engine's own, laid out [in-split][row of this part]
struct TcEngine::PartScratch {
  float *scale, *factor, *vnorm, *sval;
  int *flags;
};
TcEngine::PartScratch TcEngine::partScratch(const Run &r, int row0) {
  const size_t I = in_sizes_.size();
  PartScratch ps;
  if (r.scale != nullptr) {
    ps.scale = r.scale + row0;
    ps.factor = r.factor + row0;
    ps.vnorm = r.vnorm + row0;
    ps.sval = r.sval ? r.sval + row0 : nullptr;
    ps.flags = r.flags ? r.flags + row0 : nullptr;
  } else {
    const size_t off = I * (size_t)row0;
    ps.scale = scale_ + off;
    ps.factor = factor_ + off;
    ps.vnorm = vnorm_ + off;
    ps.sval = sval_ + off;
    ps.flags = flags_ + off;
  }
  return ps;
}

void TcEngine::launchDac(const Run &r, int row0, int rows, cudaStream_t s) {
  const int I = (int)in_sizes_.size();
  const PartScratch ps = partScratch(r, row0);
  DacParams d{};
  d.in = r.in + (long long)row0 * r.in_ss;
  d.in_ss = r.in_ss;
  d.m = rows;
  d.I = I;
  d.kpad = kpad_;
  d.insplit = (const int4 *)insplit_tab_;
  d.codes = (__nv_bfloat16 *)codes_ + (size_t)row0 * I * kpad_;
  d.codes_ld = (long long)I * kpad_;
  d.scale = ps.scale;
  d.factor = ps.factor;
  d.vnorm = ps.vnorm;
  d.sval = ps.sval;
  d.flags = ps.flags;
  d.io = r.io;
  d.alpha = r.alpha;
  d.backward = r.backward ? 1 : 0;
  d.code_bound = rintf(r.io.inp_bound / r.io.res_in);
  d.inv_res_in = 1.0f / r.io.res_in;
  if (r.gather.idx != nullptr) {
    d.in = r.in;
    d.gather = r.gather;
    d.g_row0 = row0;
    const size_t smem = (size_t)kGatherWarps * kpad_ * sizeof(float);
    if (smem > 48 * 1024 && smem > gather_smem_raised_) {
      AB200_CUDA(cudaFuncSetAttribute(dacQuantizeGatherKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
      gather_smem_raised_ = smem;
    }
    const long long warps = (long long)rows * I;
    AB200_CUDA(launchChained(dacQuantizeGatherKernel, dim3((unsigned)((warps + kGatherWarps - 1) / kGatherWarps)),
                             dim3(kGatherWarps * 32), smem, s, d));
    AB200_LAUNCH_CHECK();
    return;
  }
  bool vec = (((uintptr_t)d.in) & 15) == 0 && (r.in_ss & 3) == 0;
  for (int i = 0; i < I && vec; i++) {
    vec = (in_off_[i] & 3) == 0 && (in_sizes_[i] & 3) == 0;
  }
  if (vec && kpad_ <= 512) {
    AB200_CUDA(launchChained(dacQuantizeRowKernel, dim3((unsigned)(((long long)rows * 32 + 127) / 128)),
                             dim3(128), 0, s, d));
  } else if (vec) {
    const long long warps = (long long)rows * I;
    AB200_CUDA(launchChained(dacQuantizeLongRowKernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256),
                             0, s, d));
  } else {
    const long long warps = (long long)rows * I;
    AB200_CUDA(launchChained(dacQuantizeKernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, s, d));
  }
  AB200_LAUNCH_CHECK();
}

void TcEngine::launchMma(const Run &r0, int row0, int rows, cudaStream_t s) {
  const int I = (int)in_sizes_.size(), O = (int)out_sizes_.size();
  const PartScratch ps = partScratch(r0, row0);
  // this part as a run of its own
  Run r = r0;
  r.m = rows;
  // (a transposed store addresses by the row of the whole batch: its base stays)
  r.out = r0.out ? (r0.out_t_rows > 0 ? r0.out : r0.out + (long long)row0 * r0.out_ss) : nullptr;
  void *codes_part = (__nv_bfloat16 *)codes_ + (size_t)row0 * I * kpad_;
  struct {
    float *scale, *factor, *vnorm;
    int *flags;
  } d{ps.scale, ps.factor, ps.vnorm, ps.flags};

  CUtensorMap tm_a = makeMap(codes_part, (uint64_t)r.m, (uint64_t)I * kpad_, (uint64_t)I * kpad_);
  CUtensorMap tm_bhi = makeMap(op_hi_, (uint64_t)I * nrows_pad_, (uint64_t)kpad_, (uint64_t)kpad_);
  CUtensorMap tm_blo = makeMap(op_lo_, (uint64_t)I * nrows_pad_, (uint64_t)kpad_, (uint64_t)kpad_);

  TcKernelParams p{};
  p.m = r.m;
  p.I = I;
  p.O = O;
  p.n_chunks = n_chunks_;
  p.nrows_pad = nrows_pad_;
  p.kpad = kpad_;
  {
    // chunks per group: weight operand of a group (hi + lo, all in-splits) about 32 MB
    const double per_chunk = (double)I * kpad_ * TC_N * 4.0;
    int g = (int)(32.0 * 1024 * 1024 / per_chunk);
    p.group = g < 1 ? 1 : (g > n_chunks_ ? n_chunks_ : g);
  }
  p.chunk = (const int4 *)chunk_tab_;
  p.insplit = (const int4 *)insplit_tab_;
  p.outn = outn_tab_;
  p.key = r.key;
  p.call = r.call;
  p.noise_id0 = r.noise_id0;
  p.noise_stride = r.noise_stride > 0 ? r.noise_stride : O;
  p.scale = d.scale;
  p.factor = d.factor;
  p.vnorm = d.vnorm;
  p.tile_scale = r.tile_scale;
  p.bias = r.bias;
  p.flags = r.io.bm != AB200_BM_NONE ? d.flags : nullptr;
  p.out = r.out;
  p.out_ss = r.out_ss;
  p.out_table = r.out_table;
  p.code_table = r.code_table;
  p.fac_table = r.fac_table;
  const bool codes = r.code_table != nullptr;
  if (codes) {
    if (!codesSupported(r.io) || r.fac_table == nullptr || r.tile_scale != nullptr ||
        r.bias != nullptr || r.accumulate || r.backward || r.rows_per_owner <= 0 ||
        (r.rows_per_owner & 31) != 0 || (r.out_ss & 31) != 0) {
      AB200_FATAL("tensor-core MVM: settings not eligible for the scatter of ADC codes");
    }
    for (int n : out_sizes_) {
      if ((n % TC_N) != 0) {
        AB200_FATAL("tensor-core MVM: the scatter of ADC codes needs out-splits that are multiples of 128");
      }
    }
  }
  p.rows_per_owner = r.rows_per_owner > 0 ? r.rows_per_owner : 1;
  p.row_base = row0 + r.row_base;
  p.n_owners = r.n_owners > 0 ? r.n_owners : 1;
  p.owner_blk = r.owner_block_rows;
  if (r.owner_block_rows < 0 || (r.owner_block_rows & 31) != 0) {
    AB200_FATAL("tensor-core MVM: owner blocks must be a multiple of 32 rows");
  }
  p.flag_table = r.flag_table;
  p.epoch = r.epoch;
  if (r.flag_table != nullptr) {
    if (!done_ctr_) {
      AB200_CUDA(cudaMalloc(&done_ctr_, sizeof(int)));
      AB200_CUDA(cudaMemset(done_ctr_, 0, sizeof(int)));
    }
    p.done_ctr = done_ctr_;
  }
  {
    const int rows_item = pair_rows(r.m);
    const int n_rb_items = (r.m + rows_item - 1) / rows_item;
    p.rb_rotate = n_rb_items > 0 ? ((r.rotate_rows / rows_item) % n_rb_items + n_rb_items) % n_rb_items : 0;
  }
  p.accumulate = r.accumulate ? 1 : 0;
  p.backward = r.backward ? 1 : 0;
  {
    // on unless switched off for an A/B run: measured faster on narrow and on wide outputs alike
    // (2 % on a 4096-wide layer with eight in-splits, 20 % where the output is nine times as wide
    // as the input)
    static const bool off = [] {
      const char *e = getenv("AB200_TC_ROW_STORES");
      return e && e[0] == '0';
    }();
    p.row_stores = (!off && !codes && r.out_table == nullptr && !r.accumulate && r.out_t_rows <= 0) ? 1 : 0;
  }
  p.out_t_rows = r.out_t_rows > 0 ? r.out_t_rows : 0;
  if (p.out_t_rows > 0 && (codes || r.out_table != nullptr || r.accumulate)) {
    AB200_FATAL("tensor-core MVM: a transposed output can neither be scattered nor accumulated into");
  }
  p.io = r.io;
  p.status = status_dev_;
  static const bool prof_on = getenv("AB200_TC_PROFILE") != nullptr;
  long long *prof_dev = nullptr;
  if (prof_on) {
    AB200_CUDA(cudaMalloc(&prof_dev, 148 * 8 * sizeof(long long) * 2));
    AB200_CUDA(cudaMemsetAsync(prof_dev, 0, 148 * 8 * sizeof(long long) * 2, s));
  }
  p.prof = prof_dev;
  int grid_x = 0;
  if (n_sm_ == 0) {
    AB200_CUDA(cudaDeviceGetAttribute(&n_sm_, cudaDevAttrMultiProcessorCount, device_));
  }
  const int n_sm = n_sm_;
  // the dynamic shared memory limit of a kernel variant is raised once per device
  auto raiseSmem = [&](auto kernel, int variant, int bytes) {
    if (!(smem_raised_ & (1u << variant))) {
      AB200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
      smem_raised_ |= 1u << variant;
    }
  };
  // chained with the kernels around it (see launchChained); not when the kernel signals peers
  const bool chained = pdlEnabled() && p.flag_table == nullptr;
  const bool pair = usePairs(r.m);
  const bool bm = r.io.bm != AB200_BM_NONE;
  const bool line = r.onv != nullptr;
  if (line && (codes || in_sizes_.size() != 1 || out_sizes_.size() != 1)) {
    AB200_FATAL("tensor-core MVM: a noise table per output line needs a single tile and fp32 outputs");
  }
  p.onv = r.onv;
  if (pair) {
    const int n_items = n_chunks_ * ((r.m + 2 * TC_M - 1) / (2 * TC_M));
    const int n_pairs = n_items < n_sm / 2 ? n_items : n_sm / 2;
    auto kernel = codes ? mvmTcKernel<false, true, true>
                        : line ? (bm ? mvmTcKernel<true, true, false, true> : mvmTcKernel<false, true, false, true>)
                               : (bm ? mvmTcKernel<true, true> : mvmTcKernel<false, true>);
    raiseSmem(kernel, codes ? 0 : (bm ? 1 : 2) + (line ? 6 : 0), TC2_SMEM_BYTES);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * n_pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = TC2_SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained ? 2 : 1;
    AB200_CUDA(cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_bhi, tm_blo, p));
    grid_x = 2 * n_pairs;
  } else {
    const int n_items = n_chunks_ * ((r.m + TC_M - 1) / TC_M);
    dim3 grid(n_items < n_sm ? n_items : n_sm); // one persistent CTA per SM
    auto kernel = codes ? mvmTcKernel<false, false, true>
                        : line ? (bm ? mvmTcKernel<true, false, false, true> : mvmTcKernel<false, false, false, true>)
                               : (bm ? mvmTcKernel<true, false> : mvmTcKernel<false, false>);
    raiseSmem(kernel, codes ? 3 : (bm ? 4 : 5) + (line ? 6 : 0), TC_SMEM_BYTES);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = TC_SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained ? 1 : 0;
    AB200_CUDA(cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_bhi, tm_blo, p));
    grid_x = (int)grid.x;
  }
  AB200_LAUNCH_CHECK();
  if (prof_on) {
    // diagnostics only: average wait cycles per role over the CTAs (synchronises)
    const int n = grid_x < 296 ? grid_x : 296;
    std::vector<long long> h((size_t)n * 8);
    AB200_CUDA(cudaStreamSynchronize(s));
    AB200_CUDA(cudaMemcpy(h.data(), prof_dev, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    cudaFree(prof_dev);
    double avg[8] = {0};
    for (int c = 0; c < n; c++) {
      for (int k = 0; k < 8; k++) {
        avg[k] += (double)h[(size_t)c * 8 + k] / n;
      }
    }
    fprintf(stderr,
            "[ab200 tc] cycles/CTA: mma total %.0f (wait operands %.0f, accumulator %.0f, issuing "
            "%.0f) | tma wait stage %.0f, issuing %.0f | epilogue total %.0f (wait accumulator "
            "%.0f)\n",
            avg[3], avg[0], avg[2], avg[1], avg[4], avg[5], avg[7], avg[6]);
  }
}

} // namespace ab200
