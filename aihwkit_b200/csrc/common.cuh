// Shared device/host helpers of the B200 analog-tile library: error handling, the
// counter-based noise generator, and the fp32 discretisation steps of the IO chain.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>

namespace ab200 {

// Errors follow the reference's convention (RPU_FATAL -> std::runtime_error,
// src/rpucuda/utility_functions.h:63-69); the C ABI turns them into return codes.
#define AB200_FATAL(msg)                                                                           \
  do {                                                                                             \
    std::ostringstream ss_;                                                                        \
    ss_ << msg;                                                                                    \
    throw std::runtime_error(ss_.str());                                                           \
  } while (0)

#define AB200_CUDA(call)                                                                           \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess) {                                                                       \
      AB200_FATAL("CUDA error " << cudaGetErrorName(e_) << " (" << cudaGetErrorString(e_)          \
                                << ") at " << __FILE__ << ":" << __LINE__);                        \
    }                                                                                              \
  } while (0)

void countLaunch(int n = 1);
#define AB200_LAUNCH_CHECK()                                                                       \
  do {                                                                                             \
    ab200::countLaunch();                                                                          \
    AB200_CUDA(cudaGetLastError());                                                                \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch for the chains of small kernels of a training step (noise
// management -> MVM -> bound-management re-run -> pulse preparation -> update): a kernel launched
// with launchChained may be scheduled while its predecessor in the stream still runs, so that its
// launch latency hides behind it. Every such kernel starts with pdlEnter(): it waits there until
// the predecessor grid has completed and its writes are visible, and then lets its own successor
// start launching. Before pdlEnter() a kernel touches no global memory. Set AB200_PDL=0 to launch
// the same kernels with plain stream order.
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void pdlEnter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif
bool pdlEnabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launchChained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdlEnabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
// The reference keeps one XORWOW state per thread in global memory
// (src/rpucuda/cuda/cuda_util.cu:163-211); here every noise sample is a pure function of
// (seed, call counter, element index, purpose tag), so no generator state is ever loaded or
// stored and the result does not depend on how the work is tiled over threads.
// ---------------------------------------------------------------------------------------------
struct PhiloxKey {
  uint32_t k0, k1;
};

template <int ROUNDS>
__host__ __device__ __forceinline__ void
philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, PhiloxKey key, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  uint32_t k0 = key.k0, k1 = key.k1;
#pragma unroll
  for (int r = 0; r < ROUNDS; r++) {
    // one widening multiply per S-box gives both halves of the product
    uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0;
    c1 = lo1;
    c2 = n2;
    c3 = lo0;
    k0 += W0;
    k1 += W1;
  }
  out[0] = c0;
  out[1] = c1;
  out[2] = c2;
  out[3] = c3;
}

// Ten rounds is the standard strength, used wherever individual bits are consumed (pulse
// trains). The Gaussian output noise of the MVM uses seven rounds, the smallest count the
// authors report as passing BigCrush; it is generated once per output element and is the
// largest arithmetic cost of the tensor-core epilogue.
__host__ __device__ __forceinline__ void
philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, PhiloxKey key, uint32_t out[4]) {
  philox4x32<10>(c0, c1, c2, c3, key, out);
}

// purpose tags (4th counter word) so that streams never overlap
enum : uint32_t {
  TAG_FWD_OUT = 0x10000000u,   // + bound-management round
  TAG_BWD_OUT = 0x20000000u,
  TAG_PULSE_X = 0x30000000u,
  TAG_PULSE_D = 0x40000000u,
  TAG_DEVICE = 0x50000000u,    // + refill ordinal
  TAG_TRANSFER_READ = 0x60000000u,
  TAG_FWD_IN = 0x70000000u,    // input noise / stochastic DAC rounding; + bound-management round
  TAG_BWD_IN = 0x80000000u,
  TAG_FWD_OUT_U = 0x90000000u, // stochastic ADC rounding; + bound-management round
  TAG_BWD_OUT_U = 0xA0000000u,
};

#ifdef __CUDACC__
// MUFU approximations in their flush-to-zero form: the arguments here are never subnormal, and
// the plain forms carry extra instructions that rescale subnormal inputs
__device__ __forceinline__ float lg2Ftz(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float cosFtz(float x) {
  float y;
  asm("cos.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sinFtz(float x) {
  float y;
  asm("sin.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// uniform in (0,1) with 24 random bits
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

// Two standard normals from two 32-bit words (Box-Muller). The uniforms are built from the top
// 23 bits by setting the exponent, which keeps the integer-to-float conversions off the
// quarter-rate conversion pipe; u1 lies in [2^-23, 1], so the radius is finite (<= 5.65).
__device__ __forceinline__ void boxMuller(uint32_t a, uint32_t b, float &z0, float &z1) {
  float u1 = 2.0f - __uint_as_float(0x3f800000u | (a >> 9));
  float u2 = __uint_as_float(0x3f800000u | (b >> 9)) - 1.0f;
  float r2 = -1.3862943611198906f * __log2f(u1); // -2 ln(u1)
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(r2));
  float ang = 6.283185307179586f * u2;
  z0 = r * __cosf(ang);
  z1 = r * __sinf(ang);
}

// Two standard normals from ONE 32-bit word, 16 bits each for radius and angle (the MVM output
// noise draws one Gaussian per output element and in-split; the generator is the largest
// arithmetic cost of the epilogue). A byte permute
// drops a half-word into the low mantissa bits of 1.0f (f = 1 + X * 2^-23), and one FMA each maps
// that to u1 = 1 - X * 2^-16 in [2^-16, 1] (radius up to 4.71) and to the angle 2 pi X * 2^-16.
__device__ __forceinline__ void boxMuller16(uint32_t a, float &z0, float &z1) {
  const float fr = __uint_as_float(__byte_perm(a, 0x3f800000u, 0x7632));
  const float fa = __uint_as_float(__byte_perm(a, 0x3f800000u, 0x7610));
  const float u1 = fmaf(fr, -128.0f, 129.0f);
  const float ang = fmaf(fa, 804.24771931898703f, -804.24771931898703f); // 2 pi * 128 * (f - 1)
  const float r2 = -1.3862943611198906f * lg2Ftz(u1); // -2 ln(u1)
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(r2));
  z0 = r * cosFtz(ang);
  z1 = r * sinFtz(ang);
}

// four standard normals for noise block `blk` of call `call`; a block covers four consecutive
// output columns of one row and uses words 0 and 1 (even blocks) or 2 and 3 (odd blocks) of the
// Philox output of block pair blk / 2
__device__ __forceinline__ void
gauss4(PhiloxKey key, uint64_t blk, uint32_t call, uint32_t tag, float z[4]) {
  uint32_t r[4];
  const uint64_t pair = blk >> 1;
  philox4x32<7>((uint32_t)pair, (uint32_t)(pair >> 32), call, tag, key, r);
  const bool odd = (blk & 1) != 0;
  boxMuller16(odd ? r[2] : r[0], z[0], z[1]);
  boxMuller16(odd ? r[3] : r[1], z[2], z[3]);
}

// eight standard normals for the block pair `pair` (blocks 2 * pair and 2 * pair + 1 of gauss4)
__device__ __forceinline__ void
gauss8(PhiloxKey key, uint64_t pair, uint32_t call, uint32_t tag, float z[8]) {
  uint32_t r[4];
  philox4x32<7>((uint32_t)pair, (uint32_t)(pair >> 32), call, tag, key, r);
  boxMuller16(r[0], z[0], z[1]);
  boxMuller16(r[1], z[2], z[3]);
  boxMuller16(r[2], z[4], z[5]);
  boxMuller16(r[3], z[6], z[7]);
}

// ---- generator of the tensor-core epilogue: the same Philox4x32-7 stream, lean in instructions ----
// Round keys of one launch, computed once (the key is the same for every draw of a launch).
struct Philox7Keys {
  uint32_t a[7], b[7];
};
__device__ __forceinline__ Philox7Keys philox7Keys(PhiloxKey key) {
  Philox7Keys k;
#pragma unroll
  for (int r = 0; r < 7; r++) {
    k.a[r] = key.k0 + (uint32_t)r * 0x9E3779B9u;
    k.b[r] = key.k1 + (uint32_t)r * 0xBB67AE85u;
  }
  return k;
}
__device__ __forceinline__ void
philox7Keyed(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const Philox7Keys &k, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
#pragma unroll
  for (int r = 0; r < 7; r++) {
    const uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k.a[r], n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k.b[r];
    c0 = n0;
    c1 = (uint32_t)p1;
    c2 = n2;
    c3 = (uint32_t)p0;
  }
  out[0] = c0;
  out[1] = c1;
  out[2] = c2;
  out[3] = c3;
}
// eight standard normals of noise block pair `pair` (64-bit ordinal) of call `call`
__device__ __forceinline__ void
gauss8Keyed(const Philox7Keys &k, uint64_t pair, uint32_t call, uint32_t tag, float z[8]) {
  uint32_t r[4];
  philox7Keyed((uint32_t)pair, (uint32_t)(pair >> 32), call, tag, k, r);
  boxMuller16(r[0], z[0], z[1]);
  boxMuller16(r[1], z[2], z[3]);
  boxMuller16(r[2], z[4], z[5]);
  boxMuller16(r[3], z[6], z[7]);
}

// getDiscretizedValueSR<false> (src/rpucuda/utility_functions.h:204-210): rint(v / res) * res with
// round-half-to-even, as separate correctly-rounded fp32 operations (no FMA contraction).
__device__ __forceinline__ float discretize(float v, float res) {
  return res > 0.0f ? __fmul_rn(rintf(__fdiv_rn(v, res)), res) : v;
}
#endif

} // namespace ab200
