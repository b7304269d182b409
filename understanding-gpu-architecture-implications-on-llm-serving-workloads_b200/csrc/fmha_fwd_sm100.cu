// Fused multi-head attention forward for sm_100a:
//   O = softmax(Q K^T * scale + mask) V, online softmax in fp32, causal mask, GQA.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the keys in
// blocks of 128:
//   warps 0-3   softmax group of tile 0 (thread = query row = TMEM lane)
//   warps 4-7   softmax group of tile 1
//   warp  8     TMA loader: Q tiles once, K and V blocks through 2-deep rings
//   warps 10-11 idle (they complete the third warpgroup so that it can hand most of its
//               registers to the softmax warpgroups with setmaxnreg: 56 vs 224 per thread)
//   warp  9     MMA issuer: S_i = Q_i K_j^T (both operands K-major) into TMEM, then
//               O_i += P_i V_j with P_i read from TMEM and V_j as an MN-major
//               shared-memory operand (V is [kv, d] with d contiguous)
// While one tile's softmax runs on the CUDA cores the tensor core works on the
// other tile.  A softmax thread loads its whole S row with tcgen05.ld, takes the
// row max, rescales O in TMEM only when the max grew by more than 2^8 (the
// stale max is exact algebra: numerator and denominator carry the same factor),
// writes P = exp2(s*scale*log2e - m) as 16-bit pairs over the S columns and adds
// the row sum.  The MUFU delivers only 16 exponentials per clock per SM, which makes one
// softmax pass about as long as the two MMAs of a tile; a quarter of the exponentials
// therefore runs as a polynomial on the FMA pipe (measured +3 %; a half costs more issue
// slots than it frees MUFU cycles).  P reaches the MMA warp in two halves of 64 keys, so the first
// half of the PV product overlaps the second half of the exponentials.  The epilogue scales O by 1/l,
// stages it in the (now free) Q tile and stores it with TMA, which also clips the ragged last tile.
// Two kernels share this design: one work item per CTA (fmha_fwd_kernel, default for kv_len > 4096)
// and a persistent one (fmha_fwd_persistent_kernel, further down, default up to 4096).
//
// Reference semantics: kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_2_nv.cu
// (:36-48 GQA + offsets, :93-97 causal block range, :177-185 mask + scale,
// :188-208 recurrences, :283 final O/l) and manual/fmha_5_nv.cu:25-133.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>
#ifdef B200K_FMHA_STAMPS
#include <stdio.h>
#endif

#include "host_common.h"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kFmhaThreads = 384;  // 2 softmax warpgroups + 1 warpgroup holding the TMA and MMA warps
constexpr int kTile = 128;  // query rows per tile and keys per block
constexpr float kRescaleThreshold = 8.0f;
constexpr int kDefaultEmu = 2;  // of every 8 score pairs, how many exponentials run on the FMA pipe
// Register split by role (setmaxnreg).  setmaxnreg.inc waits until the CTA's pool - the registers it
// was launched with: threads x the per-thread count ptxas chose under __launch_bounds__, a multiple
// of 8 - has room, and waits for ever if the roles' claims add up to more than that pool, so every
// split is checked against it at compile time.
constexpr int kAuxRegs = 56, kSoftmaxRegs = 224;
constexpr int launch_regs(int threads) { return 65536 / threads / 8 * 8 > 255 ? 255 : 65536 / threads / 8 * 8; }
static_assert(256 * kSoftmaxRegs + 128 * kAuxRegs <= kFmhaThreads * launch_regs(kFmhaThreads),
              "one-item kernel: register claims exceed the launch pool");
#ifndef B200K_FMHA_P_PARTS
#define B200K_FMHA_P_PARTS 2
#endif
#ifndef B200K_FMHA_MAX_CHAINS
#define B200K_FMHA_MAX_CHAINS 4  // independent dependency chains of the row maximum (4 or 8)
#endif
// Cycle stamps of the softmax threads' phases (-DB200K_FMHA_STAMPS: a diagnostic build of the one-item kernel;
// one CTA prints, for thread 0 of each softmax group, the cycles per key block it spent in each phase).
// Without the macro every call is empty.
struct PhaseStamps {
#ifdef B200K_FMHA_STAMPS
  long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long last = 0;
  __device__ __forceinline__ void start() { last = clock64(); }
  __device__ __forceinline__ void mark(int i) {
    const long long t = clock64();
    acc[i] += t - last;
    last = t;
  }
#else
  __device__ __forceinline__ void start() {}
  __device__ __forceinline__ void mark(int) {}
#endif
};
// P is handed to the MMA warp in kPParts pieces (1, 2 or 4) of 128 / kPParts keys, so that the PV
// product of the first pieces runs while the softmax group still exponentiates the later ones.
// Two pieces by default; four in the one-item kernel at d = 128, where only the last piece's PV product (128
// instead of 256 tensor-pipe cycles) then stands between a group's hand-over and the next block's QK^T: measured
// +1..2 % at s = 8192 (full 1182-1197 -> 1202-1239 TFLOP/s, causal 1112-1114 -> 1121-1133, three alternating runs);
// the persistent kernel (within +-1 %) and d = 64 (-2 %) keep two.
static_assert(B200K_FMHA_P_PARTS == 1 || B200K_FMHA_P_PARTS == 2 || B200K_FMHA_P_PARTS == 4,
              "P is handed over in 1, 2 or 4 pieces");
template <int D, bool PERSISTENT>
constexpr int kPPartsOf = (D == 128 && !PERSISTENT && B200K_FMHA_P_PARTS == 2) ? 4 : B200K_FMHA_P_PARTS;

// Row sums on the tensor pipe (head dimension 64 only, where TMEM has 128 spare columns): every V
// stage is followed by a 64-wide box filled with ones, the PV product runs with N = D + 16, and the 16
// extra accumulator columns of a row all hold sum_k P[row][k] - the softmax denominator, summed from the
// same rounded P that multiplies V and rescaled together with O.  The softmax threads then issue no
// additions for it (a score costs about 6 issue cycles; the sum was one of them).
// Used by the one-item-per-CTA kernel (measured +4 % at d = 64, +10 % together with 3 of 8 exponentials
// emulated); the persistent kernel, whose items are short, measured 1-6 % slower with it (the PV
// product is a quarter longer) and keeps the sums in registers.
// Decoupled score and probability buffers (head dimension 64 only).  With P written over the S columns
// it came from, the next block's QK^T of a tile can only be issued after this block's PV product has
// consumed P, so a tile's chain per block is softmax -> PV -> QK^T -> softmax and its softmax group
// idles while the tensor pipe works for it (at d = 64 it waited for S a quarter to a third of the time).
// At d = 64 the two O accumulators take 2 x 64 columns, which leaves room for P buffers of their own
// (S0, S1, O0, O1, P0, P1 = 128 + 128 + 64 + 64 + 64 + 64 = 512): the MMA warp then issues S(j+1) of a
// tile as soon as its softmax group has pulled S(j) into registers, and the group goes from block to
// block without waiting for the tensor pipe.  Two more barriers per tile carry the new hazards:
// `s_free` (S columns may be overwritten) and `p_free` (PV(j) has read P(j): P(j+1) may be stored, and O
// may be rescaled - with S(j+1) issued ahead of PV(j), a finished S no longer implies a finished PV).
template <int D>
constexpr bool kCanSplitP = D == 64;
template <int D, bool PERSISTENT>
constexpr bool kHasOnesBox = D == 64 && !PERSISTENT;  // shared-memory layout: a ones box behind every V stage
template <int D, bool PERSISTENT, bool SPLITP>
constexpr bool kSumOnTensor = kHasOnesBox<D, PERSISTENT> && !SPLITP;  // its 16 extra O columns do not fit beside P0, P1
template <int D, bool PERSISTENT, bool SPLITP>
constexpr uint32_t kOCols = D + (kSumOnTensor<D, PERSISTENT, SPLITP> ? 16 : 0);  // accumulator columns of one tile

template <int D>
struct FmhaSmem {
  static constexpr uint32_t kTileBytes = kTile * D * 2;  // one Q tile, K block or V block
  static constexpr uint32_t kHalfBytes = kTile * 128;    // one 64-wide (128-byte) column box
  static constexpr uint32_t kVStride = kTileBytes + (kHasOnesBox<D, false> ? kHalfBytes : 0);  // V stage (+ ones box)
  static constexpr uint32_t kQOff = 0;
  static constexpr uint32_t kKOff = 2 * kTileBytes;
  static constexpr uint32_t kVOff = 4 * kTileBytes;
  static constexpr uint32_t kBarOff = kVOff + 2 * kVStride;
  static constexpr uint32_t kTotal = kBarOff + 256 + 1024;
};

// fills the ones boxes behind both V stages (all threads of the CTA, before the roles split)
template <int D, bool BF16, bool PERSISTENT, typename L>
__device__ __forceinline__ void fill_ones_boxes(uint8_t* smem) {
  if constexpr (kHasOnesBox<D, PERSISTENT>) {
    const uint32_t one2 = BF16 ? 0x3f803f80u : 0x3c003c00u;
    const uint4 w = make_uint4(one2, one2, one2, one2);
    for (int s = 0; s < 2; ++s) {
      uint4* box = reinterpret_cast<uint4*>(smem + L::kVOff + s * L::kVStride + L::kTileBytes);
      for (uint32_t t = threadIdx.x; t < L::kHalfBytes / 16; t += blockDim.x) box[t] = w;
    }
    fence_proxy_async_smem();  // read by the tensor core through the async proxy
  }
}

struct FmhaParams {
  int B, Hq, Hkv, Sq;
  int kv_len;      // valid keys (<= Skv); the K/V tensor maps end there
  int causal;
  int num_pairs;   // ceil(Sq / 256)
  int head_major;  // CTA order: 0 = heaviest tile pairs of all heads first, 1 = all pairs of a head together
  float scale_log2;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// packed fp32 pairs (one instruction for two lanes of a row)
__device__ __forceinline__ uint64_t f2pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2unpack(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for a pair of lanes on the FMA and integer pipes instead of the MUFU (which delivers only
// 16 results per clock per SM: at one exponential per score it would be as busy as the tensor
// pipe).  x = n + r with n = round(x), r in [-0.5, 0.5]; 2^r by a degree-3 minimax polynomial
// (relative error 7.5e-5, below the half-ulp 4.9e-4 of the 16-bit P it is rounded to); 2^n is
// added into the exponent field.  x is clamped at -125 so the exponent cannot wrap.
__device__ __forceinline__ void ex2_emulated(uint64_t x2, float& p0, float& p1) {
  float x0, x1;
  f2unpack(x2, x0, x1);
  x0 = fmaxf(x0, -125.f);
  x1 = fmaxf(x1, -125.f);
  x2 = f2pack(x0, x1);
  const uint64_t magic = f2pack(12582912.f, 12582912.f);  // 1.5 * 2^23: forces rounding to an integer
  const uint64_t j2 = add2(x2, magic);
  const uint64_t n2 = add2(j2, f2pack(-12582912.f, -12582912.f));
  const uint64_t r2 = fma2(n2, f2pack(-1.f, -1.f), x2);
  uint64_t q2 = fma2(r2, f2pack(0.0551716648f, 0.0551716648f), f2pack(0.2426111251f, 0.2426111251f));
  q2 = fma2(q2, r2, f2pack(0.6932609677f, 0.6932609677f));
  q2 = fma2(q2, r2, f2pack(0.9999280572f, 0.9999280572f));
  float q0, q1, j0, j1;
  f2unpack(q2, q0, q1);
  f2unpack(j2, j0, j1);
  // the low mantissa bits of j hold n; (j << 23) drops the magic constant's own bits
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(j0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(j1) << 23));
}

template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// One 128-key block of the online softmax for one query row (one thread): S row from TMEM ->
// P = 2^(S*scale - m) as 16-bit pairs over the same TMEM columns, handed to the MMA warp in kPParts
// pieces; l and m are the running row sum and the maximum in use.  Rescaling is lazy: m moves (and
// O and l are scaled) only when the new maximum exceeds it by more than kRescaleThreshold in some
// row of the warp, so P may reach 2^threshold.
//   lim: local index of the last visible key of this row in this block (masked = some row of the tile
//   has lim < 127); s_tmem / o_tmem: this thread's lane of the S and O accumulators.
//   SPLITP (decoupled buffers): P goes to p_tmem instead of over S; once the row is in registers the
//   group releases the S columns (`s_free_i`, when another block follows), and it waits for the previous
//   block's PV product (`p_free_i`, parity `p_free_phase`, when `wait_p_free`) before it rescales O or
//   stores the first P.  Returns false if that wait ran out.
template <int D, bool BF16, int EMU, bool SUMTC, bool SPLITP, int kPParts>
__device__ __forceinline__ bool softmax_block(uint32_t s_tmem, uint32_t p_tmem, uint32_t o_tmem, bool first,
                                              bool masked, int lim, float sc, float& m_use, float& l,
                                              uint64_t* p_part_i, uint64_t* p_ready_i, uint64_t* s_free_i,
                                              bool signal_s_free, uint64_t* p_free_i, bool wait_p_free,
                                              uint32_t p_free_phase, PhaseStamps& stamps) {
  uint32_t s[128];
  tmem_ld32(s_tmem + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
  tmem_ld32(s_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
  tmem_ld32(s_tmem + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
  tmem_ld32(s_tmem + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
  tmem_ld_wait();
  stamps.mark(1);  // S row in registers
  bool ok = true;
  if constexpr (SPLITP) {
    if (signal_s_free) {  // the row is in registers: the next block's scores may overwrite these columns
      tc_fence_before();
      mbar_arrive(s_free_i);
    }
  }
  bool pv_done = !SPLITP || !wait_p_free;
  auto wait_prev_pv = [&]() {
    if (!pv_done) {
      if (!mbar_wait(p_free_i, p_free_phase)) ok = false;
      tc_fence_after();
      pv_done = true;
    }
  };
  if (masked) {
#pragma unroll
    for (int k = 0; k < 128; ++k)
      if (k > lim) s[k] = 0xff800000u;  // -inf
  }
  auto row_max = [&]() {
#if B200K_FMHA_MAX_CHAINS == 8
    float mx[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) mx[c] = -INFINITY;
#pragma unroll
    for (int k = 0; k < 128; k += 16) {
#pragma unroll
      for (int c = 0; c < 8; ++c) mx[c] = max3(mx[c], __uint_as_float(s[k + 2 * c]), __uint_as_float(s[k + 2 * c + 1]));
    }
    return fmaxf(max3(mx[0], mx[1], mx[2]), fmaxf(max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * sc;
#else
    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
    for (int k = 0; k < 128; k += 8) {
      mx0 = max3(mx0, __uint_as_float(s[k + 0]), __uint_as_float(s[k + 1]));
      mx1 = max3(mx1, __uint_as_float(s[k + 2]), __uint_as_float(s[k + 3]));
      mx2 = max3(mx2, __uint_as_float(s[k + 4]), __uint_as_float(s[k + 5]));
      mx3 = max3(mx3, __uint_as_float(s[k + 6]), __uint_as_float(s[k + 7]));
    }
    return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc;
#endif
  };
  // moves m to m_new: l and the O accumulator (the PV products of the earlier blocks are complete:
  // this block's S was issued behind them) are scaled by 2^(m - m_new)
  auto rescale_to = [&](float m_new) {
    const float f = (m_new == -INFINITY) ? 1.f : ex2(m_use - m_new);
    m_use = m_new;
    l *= f;
    const uint64_t f2 = f2pack(f, f);
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(o_tmem + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float a, b;
        f2unpack(mul2(f2pack(__uint_as_float(o[e]), __uint_as_float(o[e + 1])), f2), a, b);
        o[e] = __float_as_uint(a);
        o[e + 1] = __float_as_uint(b);
      }
      tmem_st32(o_tmem + c * 32, o);
    }
    if constexpr (SUMTC) {
      // the row-sum columns behind O
      uint32_t o[16];
      tmem_ld16(o_tmem + D, o);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
      tmem_st16(o_tmem + D, o);
    }
  };
  // a quarter of the block: 32 keys -> 16 packed columns
  auto quarter = [&](int qt, uint32_t (&pk)[16], uint64_t& sum_a, uint64_t& sum_b) {
    const float neg = (m_use == -INFINITY) ? 0.f : -m_use;
    const uint64_t sc2 = f2pack(sc, sc), neg2 = f2pack(neg, neg);
#pragma unroll
    for (int e = 0; e < 16; e += 4) {
      // of every 8 score pairs the last EMU take their exponentials on the FMA pipe, the rest on the MUFU
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int k = qt * 32 + (e + g) * 2;
        const uint64_t x2 = fma2(f2pack(__uint_as_float(s[k]), __uint_as_float(s[k + 1])), sc2, neg2);
        float p0, p1;
        if (((e + g) & 7) >= 8 - EMU) {
          ex2_emulated(x2, p0, p1);
        } else {
          float x0, x1;
          f2unpack(x2, x0, x1);
          p0 = ex2(x0);
          p1 = ex2(x1);
        }
        if constexpr (!SUMTC) {
          if (g & 1)
            sum_b = add2(sum_b, f2pack(p0, p1));
          else
            sum_a = add2(sum_a, f2pack(p0, p1));
        }
        pk[e + g] = pack16<BF16>(p0, p1);
      }
    }
  };

  {
    const float m_new = fmaxf(m_use, row_max());
    if (first)
      m_use = m_new;
    else if (__any_sync(0xffffffffu, (m_new - m_use) > kRescaleThreshold)) {
      wait_prev_pv();  // O must hold every earlier product before it is scaled
      rescale_to(m_new);
    }
  }
  stamps.mark(2);  // mask, row maximum, vote (and the rare rescale)
  uint64_t sum_a = f2pack(0.f, 0.f), sum_b = f2pack(0.f, 0.f);
#pragma unroll
  for (int qt = 0; qt < 4; ++qt) {
    uint32_t pk[16];
    quarter(qt, pk, sum_a, sum_b);
    if (qt == 0) {
      stamps.mark(3);  // first quarter of the exponentials
      wait_prev_pv();  // the previous block's P has been consumed
      stamps.mark(4);  // (separate P columns) wait for the previous block's PV
    }
    tmem_st16(p_tmem + qt * 16, pk);
    // hand the finished piece to the MMA warp (the last piece goes through p_ready below)
    if (qt < 3 && (qt + 1) % (4 / kPParts) == 0) {
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_part_i[((qt + 1) / (4 / kPParts) - 1) * 2]);
    }
  }
  tmem_st_wait();
  tc_fence_before();
  mbar_arrive(p_ready_i);
  stamps.mark(5);  // the other three quarters, P stores, hand-over
  if constexpr (!SUMTC) {
    float a, b;
    f2unpack(add2(sum_a, sum_b), a, b);
    l += a + b;
  }
  return ok;
}


// EMU: how many of every 8 score pairs take their exponentials on the FMA pipe (0..4).
template <int D, bool BF16, int EMU, bool SPLITP>
__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const FmhaParams p) {
  static_assert(!SPLITP || kCanSplitP<D>, "separate P buffers need the spare TMEM columns of d = 64");
  using L = FmhaSmem<D>;
  constexpr int kDBoxes = D / 64;  // 64-wide column boxes per row
  constexpr uint32_t kTmemCols = 512;
  constexpr bool kSumTc = kSumOnTensor<D, false, SPLITP>;
  constexpr uint32_t kOW = kOCols<D, false, SPLITP>;
  constexpr uint32_t kSCol0 = 0, kSCol1 = 128, kOCol0 = 256, kOCol1 = 256 + kOW;
  // P over its own S columns, or (SPLITP) in 64 columns of its own behind the accumulators
  constexpr uint32_t kPCol0 = SPLITP ? 256 + 2 * kOW : kSCol0, kPCol1 = SPLITP ? 256 + 2 * kOW + 64 : kSCol1;
  static_assert(!SPLITP || kPCol1 + 64 <= kTmemCols, "TMEM map exceeds 512 columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;        // [2]
  uint64_t* k_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2]
  uint64_t* p_ready = bars + 12;  // [2]
  uint64_t* o_full = bars + 14;   // [2]
  uint64_t* p_part = bars + 16;   // [3][2]  piece 0, 1, 2 of P stored (the last piece signals p_ready)
  uint64_t* s_free = bars + 22;   // [2]  (SPLITP) S_i is in the softmax group's registers
  uint64_t* p_free = bars + 24;   // [2]  (SPLITP) PV_i of a block has read P_i (and updated O_i)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 26);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which work item ----
  // CTA order.  When all K/V fit L2 comfortably the heaviest (latest, under the causal mask)
  // tile pairs of every head go first, which balances the tail best.  Otherwise the tile
  // pairs of one head run together (heavy first), so that the CTAs resident at one time
  // share few K/V heads and those stay in L2 instead of being re-read from HBM per pair.
  const int idx = blockIdx.x;
  int h, b, pair;
  if (p.head_major) {
    pair = p.num_pairs - 1 - idx % p.num_pairs;
    const int t = idx / p.num_pairs;
    h = t % p.Hq;
    b = t / p.Hq;
  } else {
    h = idx % p.Hq;
    const int t = idx / p.Hq;
    b = t % p.B;
    pair = p.num_pairs - 1 - t / p.B;
  }
  const int hk = h / (p.Hq / p.Hkv);
  const int off = p.kv_len - p.Sq;  // causal diagonal, aligned bottom-right
  int q0[2], nb[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    q0[i] = (pair * 2 + i) * kTile;
    valid[i] = q0[i] < p.Sq;
    int kv_hi = p.kv_len;
    if (p.causal) {
      const int last_row = min(q0[i] + kTile, p.Sq) - 1;
      kv_hi = max(0, min(p.kv_len, last_row + off + 1));
    }
    nb[i] = valid[i] ? (kv_hi + kTile - 1) / kTile : 0;
  }
  const int nb_max = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      for (int part = 0; part < 3; ++part) mbar_init(&p_part[part * 2 + i], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_free[i], 1);
    }
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 9) {
    tmem_alloc<1>(tmem_holder, kTmemCols);
    tmem_relinquish<1>();
  }
  fill_ones_boxes<D, BF16, false, L>(smem);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // programmatic dependent launch: everything above (barriers, TMEM, tensor-map prefetch) may have run while
  // the kernel before this one in the stream was still running; nothing of Q, K, V is read and nothing of O
  // written before that kernel has finished
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t tmem_base = *tmem_holder;

  if (warp >= 10) {
    // idle warps of the third warpgroup
    reg_dealloc<kAuxRegs>();
  } else if (warp == 8) {
    // ------------------------------- TMA loader -------------------------------
    reg_dealloc<kAuxRegs>();
    if (elect_one() && nb_max > 0) {
      auto load_tile = [&](const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int row, int head) {
        mbar_expect_tx(bar, L::kTileBytes);
#pragma unroll
        for (int d = 0; d < kDBoxes; ++d) tma_load_4d(dst + d * L::kHalfBytes, tm, bar, d * 64, row, head, b);
      };
      bool ok = true;
      load_tile(&tmK, smem + L::kKOff, &k_full[0], 0, hk);
      for (int i = 0; i < 2; ++i)
        if (nb[i] > 0) load_tile(&tmQ, smem + L::kQOff + i * L::kTileBytes, &q_full[i], q0[i], h);
      for (int j = 0; j < nb_max && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&v_empty[s], ph ^ 1)) {
          report_timeout(p.status, KID_FMHA, ROLE_PRODUCER);
          break;
        }
        load_tile(&tmV, smem + L::kVOff + s * L::kVStride, &v_full[s], j * kTile, hk);
        if (j + 1 < nb_max) {
          const int s1 = (j + 1) & 1;
          const uint32_t ph1 = ((j + 1) >> 1) & 1;
          if (!mbar_wait(&k_empty[s1], ph1 ^ 1)) {
            report_timeout(p.status, KID_FMHA, ROLE_PRODUCER);
            break;
          }
          load_tile(&tmK, smem + L::kKOff + s1 * L::kTileBytes, &k_full[s1], (j + 1) * kTile, hk);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -------------------------------
    reg_dealloc<kAuxRegs>();
    if (elect_one() && nb_max > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(BF16 ? 1 : 0, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_pv = make_idesc_f16(BF16 ? 1 : 0, 0, 1, kTile, kOW);
      const uint32_t q_addr = smem_u32(smem + L::kQOff);
      const uint32_t k_addr = smem_u32(smem + L::kKOff);
      const uint32_t v_addr = smem_u32(smem + L::kVOff);
      const uint32_t s_col[2] = {kSCol0, kSCol1};
      const uint32_t o_col[2] = {kOCol0, kOCol1};
      const uint32_t p_col[2] = {kPCol0, kPCol1};
      bool ok = true;
      auto fail = [&]() {
        report_timeout(p.status, KID_FMHA, ROLE_MMA);
        ok = false;
      };
      // S_i = Q_i . K_stage^T : D/16 steps; 16 d-elements = 32 bytes inside a 128-byte row,
      // the next 64-wide column box is kHalfBytes further.
      auto issue_s = [&](int i, int stage) {
        const uint32_t qa = q_addr + i * L::kTileBytes;
        const uint32_t ka = k_addr + stage * L::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * L::kHalfBytes + (kk & 3) * 32;
          umma_ss<1>(tmem_base + s_col[i], make_smem_desc_sw128(qa + o, 16, 1024),
                     make_smem_desc_sw128(ka + o, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit<1>(&s_full[i]);
      };
      // O_i += P_i . V_stage : 8 steps of 16 keys; P from TMEM (8 columns of 16-bit pairs per
      // step), V MN-major: 16 keys = 16 rows of 128 bytes; 64-wide d boxes kHalfBytes apart.
      auto issue_pv = [&](int i, int stage, bool first, int kk0, int kk1) {
        const uint32_t va = v_addr + stage * L::kVStride;
#pragma unroll
        for (int kk = kk0; kk < kk1; ++kk) {
          umma_ts(tmem_base + o_col[i], tmem_base + p_col[i] + kk * 8,
                  make_smem_desc_sw128(va + kk * 2048, L::kHalfBytes, 1024), idesc_pv,
                  (!first || kk > 0) ? 1u : 0u);
        }
      };
      // PV_i of block j as the pieces of P arrive; false if a wait ran out
      auto pv_block = [&](int i, int stage, int j) {
        constexpr int kPParts = kPPartsOf<D, false>;
        constexpr int kStepsPerPart = kTile / 16 / kPParts;
#pragma unroll
        for (int part = 0; part + 1 < kPParts; ++part) {
          if (ok && !mbar_wait(&p_part[part * 2 + i], j & 1)) fail();
          if (!ok) return;
          tc_fence_after();
          issue_pv(i, stage, j == 0, part * kStepsPerPart, (part + 1) * kStepsPerPart);
        }
        if (!mbar_wait(&p_ready[i], j & 1)) {
          fail();
          return;
        }
        tc_fence_after();
        issue_pv(i, stage, j == 0, (kPParts - 1) * kStepsPerPart, kTile / 16);
      };
      if (!mbar_wait(&k_full[0], 0)) fail();
      for (int i = 0; i < 2 && ok; ++i) {
        if (nb[i] > 0) {
          if (!mbar_wait(&q_full[i], 0)) {
            fail();
            break;
          }
          tc_fence_after();
          issue_s(i, 0);
        }
      }
      if (ok) umma_commit<1>(&k_empty[0]);
      for (int j = 0; j < nb_max && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if constexpr (SPLITP) {
          // The next block's scores first: they need K(j+1) and the S columns, which a softmax group
          // releases as soon as it holds S(j) in registers - not this block's PV products.
          if (j + 1 < nb_max) {
            const int s1 = (j + 1) & 1;
            if (!mbar_wait(&k_full[s1], ((j + 1) >> 1) & 1)) {
              fail();
              break;
            }
            for (int i = 0; i < 2 && ok; ++i) {
              if (j + 1 >= nb[i]) continue;
              if (!mbar_wait(&s_free[i], j & 1)) {
                fail();
                break;
              }
              tc_fence_after();
              issue_s(i, s1);
            }
            if (!ok) break;
            umma_commit<1>(&k_empty[s1]);
          }
          if (!mbar_wait(&v_full[s], ph)) {
            fail();
            break;
          }
          for (int i = 0; i < 2 && ok; ++i) {
            if (j >= nb[i]) continue;
            pv_block(i, s, j);
            if (!ok) break;
            if (j == nb[i] - 1)
              umma_commit<1>(&o_full[i]);
            else
              umma_commit<1>(&p_free[i]);  // the group may store P(j+1) and rescale O
          }
          if (!ok) break;
          umma_commit<1>(&v_empty[s]);
        } else {
          if (!mbar_wait(&v_full[s], ph)) {
            fail();
            break;
          }
          bool k_next_ready = false;
          for (int i = 0; i < 2 && ok; ++i) {
            if (j >= nb[i]) continue;
            pv_block(i, s, j);
            if (!ok) break;
            if (j == nb[i] - 1) umma_commit<1>(&o_full[i]);
            if (j + 1 < nb[i]) {
              const int s1 = (j + 1) & 1;
              if (!k_next_ready) {
                if (!mbar_wait(&k_full[s1], ((j + 1) >> 1) & 1)) {
                  fail();
                  break;
                }
                tc_fence_after();
                k_next_ready = true;
              }
              issue_s(i, s1);
            }
          }
          if (!ok) break;
          umma_commit<1>(&v_empty[s]);
          if (j + 1 < nb_max) umma_commit<1>(&k_empty[(j + 1) & 1]);
        }
      }
    }
  } else {
    // ----------------------------- softmax groups -----------------------------
    reg_alloc<kSoftmaxRegs>();
    const int i = warp >> 2;             // tile of this group
    const int row = threadIdx.x & 127;   // query row inside the tile = TMEM lane
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_sel + (i == 0 ? kSCol0 : kSCol1);
    const uint32_t o_tmem = tmem_base + lane_sel + (i == 0 ? kOCol0 : kOCol1);
    const uint32_t p_tmem = tmem_base + lane_sel + (i == 0 ? kPCol0 : kPCol1);
    if (valid[i]) {
      const float sc = p.scale_log2;
      const int q = q0[i] + row;
      // last visible key index for this row
      const int lim_row = p.causal ? min(q + off, p.kv_len - 1) : p.kv_len - 1;
      // smallest such index over the rows of the tile: blocks reaching beyond it have masked keys
      const int tile_min_lim = p.causal ? min(q0[i] + off, p.kv_len - 1) : p.kv_len - 1;
      float m_use = -INFINITY;
      float l = 0.f;
      bool ok = true;
      PhaseStamps stamps;
      stamps.start();
      for (int j = 0; j < nb[i]; ++j) {
        if (!mbar_wait(&s_full[i], j & 1)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        stamps.mark(0);  // wait for S
        const int k0 = j * kTile;
        if (!softmax_block<D, BF16, EMU, kSumTc, SPLITP, kPPartsOf<D, false>>(
                s_tmem, p_tmem, o_tmem, j == 0, k0 + kTile - 1 > tile_min_lim, lim_row - k0, sc, m_use, l, &p_part[i],
                &p_ready[i], &s_free[i], j + 1 < nb[i], &p_free[i], j > 0, (uint32_t)((j - 1) & 1), stamps)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_SOFTMAX);
          ok = false;
          break;
        }
      }

#ifdef B200K_FMHA_STAMPS
      if (blockIdx.x == gridDim.x / 2 && (threadIdx.x & 127) == 0 && nb[i] > 0)
        printf("stamps tile %d blocks %d: wait_S %lld ld %lld max %lld exp_q0 %lld wait_pv %lld exp_rest %lld (cycles per block)\n", i,
               nb[i], stamps.acc[0] / nb[i], stamps.acc[1] / nb[i], stamps.acc[2] / nb[i], stamps.acc[3] / nb[i],
               stamps.acc[4] / nb[i], stamps.acc[5] / nb[i]);
#endif
      // ------------------------------ epilogue ------------------------------
      if (ok && nb[i] > 0) {
        if (!mbar_wait(&o_full[i], 0)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_EPILOGUE);
          ok = false;
        }
        tc_fence_after();
      }
      if (ok) {
        if constexpr (kSumTc) {
          if (nb[i] > 0) {  // the denominator was summed by the PV products: 16 equal columns behind O
            const uint32_t t = tmem_ld1(o_tmem + D);
            tmem_ld_wait();
            l = __uint_as_float(t);
          }
        }
        // A row that saw no visible key in any block (m still -inf) is zero.  Its l is not: a masked score's
        // emulated exponential is clamped to 2^-125, which a bf16 P keeps (fp16 flushes it), so l and O hold
        // a mean of V scaled by 2^-125 that the division would blow up to a mean of V.
        const float inv = (l > 0.f && m_use != -INFINITY) ? 1.f / l : 0.f;
        uint8_t* stage = smem + L::kQOff + i * L::kTileBytes;  // Q_i is no longer read
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          if (nb[i] > 0) {
            tmem_ld32(o_tmem + c * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0u;
          }
          uint8_t* rowp = stage + (c >> 1) * L::kHalfBytes + row * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack16<BF16>(__uint_as_float(o[8 * g + 0]) * inv, __uint_as_float(o[8 * g + 1]) * inv);
            w.y = pack16<BF16>(__uint_as_float(o[8 * g + 2]) * inv, __uint_as_float(o[8 * g + 3]) * inv);
            w.z = pack16<BF16>(__uint_as_float(o[8 * g + 4]) * inv, __uint_as_float(o[8 * g + 5]) * inv);
            w.w = pack16<BF16>(__uint_as_float(o[8 * g + 6]) * inv, __uint_as_float(o[8 * g + 7]) * inv);
            const int chunk = (c & 1) * 4 + g;
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (row & 7)) << 4)) = w;
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1 + i, 128);
        if (row == 0) {
#pragma unroll
          for (int d = 0; d < kDBoxes; ++d) tma_store_4d(&tmO, stage + d * L::kHalfBytes, d * 64, q0[i], h, b);
          tma_store_commit();
          tma_store_wait_all<0>();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Persistent variant: one CTA per SM walks a list of work items (batch, head, tile pair).  TMEM,
// barriers and tensor-map prefetches are set up once; the K/V rings, the S/P handshakes and the
// Q / O hand-overs keep running across items (every barrier's phase is tracked with a running
// counter), so the loads and the first QK^T of the next item overlap the last PV and the epilogue
// of the current one.  The epilogue stages O in its own 16 KB buffer per warpgroup (64 columns at a
// time) instead of the Q tile, which the loader may already be refilling.
// ---------------------------------------------------------------------------------------------
// Register split of the persistent kernel (per thread; 256 softmax threads + 128 others must fit the
// 64K registers of the SM): its loader and MMA threads carry more running state than in the one-item kernel.
constexpr int kPersistAuxRegs = 88, kPersistSoftmaxRegs = 208;
static_assert(256 * kPersistSoftmaxRegs + 128 * kPersistAuxRegs <= kFmhaThreads * launch_regs(kFmhaThreads),
              "persistent kernel: register claims exceed the launch pool");

template <int D>
struct FmhaPSmem {
  static constexpr uint32_t kTileBytes = kTile * D * 2;
  static constexpr uint32_t kHalfBytes = kTile * 128;
  static constexpr uint32_t kQOff = 0;
  static constexpr uint32_t kKOff = 2 * kTileBytes;
  static constexpr uint32_t kVStride = kTileBytes + (kHasOnesBox<D, true> ? kHalfBytes : 0);  // V stage (+ ones box)
  static constexpr uint32_t kVOff = 4 * kTileBytes;
  static constexpr uint32_t kStageOff = kVOff + 2 * kVStride;  // 2 x 16 KB output staging
  static constexpr uint32_t kBarOff = kStageOff + 2 * kHalfBytes;
  static constexpr uint32_t kTotal = kBarOff + 256 + 1024;
};

struct FmhaItem {
  int h, b, hk;
  int q0[2], nb[2];
  bool valid[2];
  int nb_max;
};

__device__ __forceinline__ FmhaItem fmha_item(const FmhaParams& p, int idx) {
  FmhaItem it;
  int pair;
  if (p.head_major) {
    pair = p.num_pairs - 1 - idx % p.num_pairs;
    const int t = idx / p.num_pairs;
    it.h = t % p.Hq;
    it.b = t / p.Hq;
  } else {
    it.h = idx % p.Hq;
    const int t = idx / p.Hq;
    it.b = t % p.B;
    pair = p.num_pairs - 1 - t / p.B;
  }
  it.hk = it.h / (p.Hq / p.Hkv);
  const int off = p.kv_len - p.Sq;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    it.q0[i] = (pair * 2 + i) * kTile;
    it.valid[i] = it.q0[i] < p.Sq;
    int kv_hi = p.kv_len;
    if (p.causal) {
      const int last_row = min(it.q0[i] + kTile, p.Sq) - 1;
      kv_hi = max(0, min(p.kv_len, last_row + off + 1));
    }
    it.nb[i] = it.valid[i] ? (kv_hi + kTile - 1) / kTile : 0;
  }
  it.nb_max = max(it.nb[0], it.nb[1]);
  return it;
}

template <int D, bool BF16, int EMU, bool SPLITP>
__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                           const FmhaParams p, int total_items) {
  static_assert(!SPLITP || kCanSplitP<D>, "separate P buffers need the spare TMEM columns of d = 64");
  using L = FmhaPSmem<D>;
  constexpr int kDBoxes = D / 64;
  constexpr uint32_t kTmemCols = 512;
  constexpr bool kSumTc = kSumOnTensor<D, true, SPLITP>;
  constexpr uint32_t kOW = kOCols<D, true, SPLITP>;
  constexpr uint32_t kSCol0 = 0, kSCol1 = 128, kOCol0 = 256, kOCol1 = 256 + kOW;
  constexpr uint32_t kPCol0 = SPLITP ? 256 + 2 * kOW : kSCol0, kPCol1 = SPLITP ? 256 + 2 * kOW + 64 : kSCol1;
  static_assert(!SPLITP || kPCol1 + 64 <= kTmemCols, "TMEM map exceeds 512 columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;         // [2]  Q_i landed
  uint64_t* q_free = bars + 2;     // [2]  every S MMA of the item has read Q_i
  uint64_t* k_full = bars + 4;     // [2]
  uint64_t* k_empty = bars + 6;    // [2]
  uint64_t* v_full = bars + 8;     // [2]
  uint64_t* v_empty = bars + 10;   // [2]
  uint64_t* s_full = bars + 12;    // [2]
  uint64_t* p_ready = bars + 14;   // [2]
  uint64_t* o_full = bars + 16;    // [2]  last PV of the item done
  uint64_t* o_free = bars + 18;    // [2]  epilogue has read O_i out of TMEM
  uint64_t* p_part = bars + 20;    // [3][2]  piece 0, 1, 2 of P stored (the last piece signals p_ready)
  uint64_t* s_free = bars + 26;    // [2]  (SPLITP) S_i is in the softmax group's registers
  uint64_t* p_free = bars + 28;    // [2]  (SPLITP) PV_i of a block has read P_i (and updated O_i)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 30);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Items are ordered heavy to light; round r hands items [r*G, (r+1)*G) to the G CTAs forwards on
  // even rounds and backwards on odd ones, which evens out linearly decreasing work.
  auto snake_item = [&](int r) {
    const int g = (int)gridDim.x;
    return r * g + ((r & 1) ? g - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_free[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      for (int part = 0; part < 3; ++part) mbar_init(&p_part[part * 2 + i], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_free[i], 128);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_free[i], 1);
    }
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 9) {
    tmem_alloc<1>(tmem_holder, kTmemCols);
    tmem_relinquish<1>();
  }
  fill_ones_boxes<D, BF16, true, L>(smem);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_launch_dependents();  // programmatic dependent launch, as in the one-item kernel
  grid_dependency_wait();
  const uint32_t tmem_base = *tmem_holder;

  if (warp >= 10) {
    reg_dealloc<kPersistAuxRegs>();
  } else if (warp == 8) {
    // ------------------------------- TMA loader -------------------------------
    reg_dealloc<kPersistAuxRegs>();
    if (elect_one()) {
      uint32_t kc = 0, vc = 0, qn[2] = {0, 0};
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int row, int head, int b) {
        mbar_expect_tx(bar, L::kTileBytes);
#pragma unroll
        for (int d = 0; d < kDBoxes; ++d) tma_load_4d(dst + d * L::kHalfBytes, tm, bar, d * 64, row, head, b);
      };
      auto load_k = [&](const FmhaItem& it, int j) {
        const uint32_t st = kc & 1;
        if (!mbar_wait(&k_empty[st], ((kc >> 1) & 1) ^ 1)) {
          report_timeout(p.status, KID_FMHA, ROLE_PRODUCER);
          ok = false;
          return;
        }
        load_tile(&tmK, smem + L::kKOff + st * L::kTileBytes, &k_full[st], j * kTile, it.hk, it.b);
        ++kc;
      };
      for (int r = 0; r * (int)gridDim.x < total_items && ok; ++r) {
        const int w = snake_item(r);
        if (w >= total_items) continue;
        const FmhaItem it = fmha_item(p, w);
        if (it.nb_max == 0) continue;
        load_k(it, 0);
        for (int i = 0; i < 2 && ok; ++i) {
          if (it.nb[i] == 0) continue;
          if (!mbar_wait(&q_free[i], (qn[i] & 1) ^ 1)) {
            report_timeout(p.status, KID_FMHA, ROLE_PRODUCER);
            ok = false;
            break;
          }
          load_tile(&tmQ, smem + L::kQOff + i * L::kTileBytes, &q_full[i], it.q0[i], it.h, it.b);
          ++qn[i];
        }
        for (int j = 0; j < it.nb_max && ok; ++j) {
          const uint32_t st = vc & 1;
          if (!mbar_wait(&v_empty[st], ((vc >> 1) & 1) ^ 1)) {
            report_timeout(p.status, KID_FMHA, ROLE_PRODUCER);
            ok = false;
            break;
          }
          load_tile(&tmV, smem + L::kVOff + st * L::kVStride, &v_full[st], j * kTile, it.hk, it.b);
          ++vc;
          if (j + 1 < it.nb_max) load_k(it, j + 1);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -------------------------------
    reg_dealloc<kPersistAuxRegs>();
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_f16(BF16 ? 1 : 0, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_pv = make_idesc_f16(BF16 ? 1 : 0, 0, 1, kTile, kOW);
      const uint32_t q_addr = smem_u32(smem + L::kQOff);
      const uint32_t k_addr = smem_u32(smem + L::kKOff);
      const uint32_t v_addr = smem_u32(smem + L::kVOff);
      const uint32_t s_col[2] = {kSCol0, kSCol1};
      const uint32_t o_col[2] = {kOCol0, kOCol1};
      const uint32_t p_col[2] = {kPCol0, kPCol1};
      uint32_t kc = 0, vc = 0, qn[2] = {0, 0}, pn[2] = {0, 0}, on[2] = {0, 0}, sfn[2] = {0, 0};
      bool ok = true;
      auto fail = [&]() {
        report_timeout(p.status, KID_FMHA, ROLE_MMA);
        ok = false;
      };
      auto issue_s = [&](int i, uint32_t stage) {
        const uint32_t qa = q_addr + i * L::kTileBytes;
        const uint32_t ka = k_addr + stage * L::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * L::kHalfBytes + (kk & 3) * 32;
          umma_ss<1>(tmem_base + s_col[i], make_smem_desc_sw128(qa + o, 16, 1024),
                     make_smem_desc_sw128(ka + o, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit<1>(&s_full[i]);
      };
      auto issue_pv = [&](int i, uint32_t stage, bool first, int kk0, int kk1) {
        const uint32_t va = v_addr + stage * L::kVStride;
#pragma unroll
        for (int kk = kk0; kk < kk1; ++kk) {
          umma_ts(tmem_base + o_col[i], tmem_base + p_col[i] + kk * 8,
                  make_smem_desc_sw128(va + kk * 2048, L::kHalfBytes, 1024), idesc_pv,
                  (!first || kk > 0) ? 1u : 0u);
        }
      };
      // PV_i of block j of the item as the pieces of P arrive (the item's first one also waits until the
      // previous item's O_i has been read out); ok turns false if a wait ran out
      auto pv_block = [&](int i, int j) {
        if (j == 0 && !mbar_wait(&o_free[i], (on[i] & 1) ^ 1)) {
          fail();
          return;
        }
        constexpr int kPParts = kPPartsOf<D, true>;
        constexpr int kStepsPerPart = kTile / 16 / kPParts;
#pragma unroll
        for (int part = 0; part + 1 < kPParts; ++part) {
          if (ok && !mbar_wait(&p_part[part * 2 + i], pn[i] & 1)) fail();
          if (!ok) return;
          tc_fence_after();
          issue_pv(i, vc & 1, j == 0, part * kStepsPerPart, (part + 1) * kStepsPerPart);
        }
        if (!mbar_wait(&p_ready[i], pn[i] & 1)) {
          fail();
          return;
        }
        ++pn[i];
        tc_fence_after();
        issue_pv(i, vc & 1, j == 0, (kPParts - 1) * kStepsPerPart, kTile / 16);
      };
      for (int r = 0; r * (int)gridDim.x < total_items && ok; ++r) {
        const int w = snake_item(r);
        if (w >= total_items) continue;
        const FmhaItem it = fmha_item(p, w);
        if (it.nb_max == 0) continue;
        // first score block of both tiles
        if (!mbar_wait(&k_full[kc & 1], (kc >> 1) & 1)) {
          fail();
          break;
        }
        for (int i = 0; i < 2 && ok; ++i) {
          if (it.nb[i] == 0) continue;
          if (!mbar_wait(&q_full[i], qn[i] & 1)) {
            fail();
            break;
          }
          tc_fence_after();
          issue_s(i, kc & 1);
        }
        if (!ok) break;
        umma_commit<1>(&k_empty[kc & 1]);
        ++kc;
        for (int j = 0; j < it.nb_max && ok; ++j) {
          if constexpr (SPLITP) {
            // the next block's scores first (they do not depend on this block's PV products)
            if (j + 1 < it.nb_max) {
              if (!mbar_wait(&k_full[kc & 1], (kc >> 1) & 1)) {
                fail();
                break;
              }
              for (int i = 0; i < 2 && ok; ++i) {
                if (j + 1 >= it.nb[i]) continue;
                if (!mbar_wait(&s_free[i], sfn[i] & 1)) {
                  fail();
                  break;
                }
                ++sfn[i];
                tc_fence_after();
                issue_s(i, kc & 1);
                if (j + 2 == it.nb[i]) {
                  umma_commit<1>(&q_free[i]);  // that was the item's last read of Q_i
                  ++qn[i];
                }
              }
              if (!ok) break;
              umma_commit<1>(&k_empty[kc & 1]);
              ++kc;
            }
            if (!mbar_wait(&v_full[vc & 1], (vc >> 1) & 1)) {
              fail();
              break;
            }
            for (int i = 0; i < 2 && ok; ++i) {
              if (j >= it.nb[i]) continue;
              pv_block(i, j);
              if (!ok) break;
              if (j == it.nb[i] - 1) {
                umma_commit<1>(&o_full[i]);
                ++on[i];
                if (it.nb[i] == 1) {  // single-block item: the prologue's S_i was the only read of Q_i
                  umma_commit<1>(&q_free[i]);
                  ++qn[i];
                }
              } else {
                umma_commit<1>(&p_free[i]);
              }
            }
            if (!ok) break;
            umma_commit<1>(&v_empty[vc & 1]);
            ++vc;
          } else {
            if (!mbar_wait(&v_full[vc & 1], (vc >> 1) & 1)) {
              fail();
              break;
            }
            bool k_next_ready = false;
            for (int i = 0; i < 2 && ok; ++i) {
              if (j >= it.nb[i]) continue;
              pv_block(i, j);
              if (!ok) break;
              if (j == it.nb[i] - 1) {
                umma_commit<1>(&o_full[i]);
                ++on[i];
                umma_commit<1>(&q_free[i]);  // covers the item's last S_i as well
                ++qn[i];
              }
              if (j + 1 < it.nb[i]) {
                if (!k_next_ready) {
                  if (!mbar_wait(&k_full[kc & 1], (kc >> 1) & 1)) {
                    fail();
                    break;
                  }
                  tc_fence_after();
                  k_next_ready = true;
                }
                issue_s(i, kc & 1);
              }
            }
            if (!ok) break;
            umma_commit<1>(&v_empty[vc & 1]);
            ++vc;
            if (j + 1 < it.nb_max) {
              umma_commit<1>(&k_empty[kc & 1]);
              ++kc;
            }
          }
        }
      }
    }
  } else {
    // ----------------------------- softmax groups -----------------------------
    reg_alloc<kPersistSoftmaxRegs>();
    const int i = warp >> 2;
    const int row = threadIdx.x & 127;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_sel + (i == 0 ? kSCol0 : kSCol1);
    const uint32_t o_tmem = tmem_base + lane_sel + (i == 0 ? kOCol0 : kOCol1);
    const uint32_t p_tmem = tmem_base + lane_sel + (i == 0 ? kPCol0 : kPCol1);
    uint8_t* stage = smem + L::kStageOff + i * L::kHalfBytes;
    const float sc = p.scale_log2;
    const int off = p.kv_len - p.Sq;
    uint32_t sn = 0, itn = 0, pfn = 0;
    bool ok = true;
    bool store_pending = false;
    for (int r = 0; r * (int)gridDim.x < total_items && ok; ++r) {
      const int w = snake_item(r);
      if (w >= total_items) continue;
      const FmhaItem it = fmha_item(p, w);
      if (!it.valid[i]) continue;
      const int q = it.q0[i] + row;
      const int lim_row = p.causal ? min(q + off, p.kv_len - 1) : p.kv_len - 1;
      const int tile_min_lim = p.causal ? min(it.q0[i] + off, p.kv_len - 1) : p.kv_len - 1;
      float m_use = -INFINITY;
      float l = 0.f;
      PhaseStamps stamps;  // (the diagnostic build prints from the one-item kernel only)
      for (int j = 0; j < it.nb[i]; ++j) {
        if (!mbar_wait(&s_full[i], sn & 1)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_SOFTMAX);
          ok = false;
          break;
        }
        ++sn;
        tc_fence_after();
        const int k0 = j * kTile;
        if (!softmax_block<D, BF16, EMU, kSumTc, SPLITP, kPPartsOf<D, true>>(
                s_tmem, p_tmem, o_tmem, j == 0, k0 + kTile - 1 > tile_min_lim, lim_row - k0, sc, m_use, l, &p_part[i],
                &p_ready[i], &s_free[i], j + 1 < it.nb[i], &p_free[i], j > 0, pfn & 1, stamps)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_SOFTMAX);
          ok = false;
          break;
        }
        if (SPLITP && j > 0) ++pfn;
      }
      if (!ok) break;

      // ------------------------------ epilogue ------------------------------
      const bool have_o = it.nb[i] > 0;
      if (have_o) {
        if (!mbar_wait(&o_full[i], itn & 1)) {
          if (lane == 0) report_timeout(p.status, KID_FMHA, ROLE_EPILOGUE);
          ok = false;
          break;
        }
        ++itn;
        tc_fence_after();
        if constexpr (kSumTc) {  // the denominator was summed by the PV products
          const uint32_t t = tmem_ld1(o_tmem + D);
          tmem_ld_wait();
          l = __uint_as_float(t);
        }
      }
      // (a row without any visible key is zero: see the one-item kernel's epilogue)
      const float inv = (l > 0.f && m_use != -INFINITY) ? 1.f / l : 0.f;
#pragma unroll
      for (int hb = 0; hb < kDBoxes; ++hb) {
        // 64 columns of O at a time: TMEM -> registers -> staging buffer -> TMA store
        uint32_t o[64];
        if (have_o) {
          tmem_ld32(o_tmem + hb * 64, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
          tmem_ld32(o_tmem + hb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32]));
          tmem_ld_wait();
          if (hb == kDBoxes - 1) {
            tc_fence_before();
            mbar_arrive(&o_free[i]);  // all of O_i is in registers: the next item's first PV may overwrite it
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; ++e) o[e] = 0u;
        }
        // the previous TMA store out of this staging buffer must have finished reading it
        if (store_pending) {
          if (row == 0) tma_store_wait_read<0>();
          named_barrier_sync(1 + i, 128);
        }
        uint8_t* rowp = stage + row * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int e = g * 8;
          uint4 wv;
          wv.x = pack16<BF16>(__uint_as_float(o[e + 0]) * inv, __uint_as_float(o[e + 1]) * inv);
          wv.y = pack16<BF16>(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
          wv.z = pack16<BF16>(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
          wv.w = pack16<BF16>(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
          *reinterpret_cast<uint4*>(rowp + ((g ^ (row & 7)) << 4)) = wv;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1 + i, 128);
        if (row == 0) {
          tma_store_4d(&tmO, stage, hb * 64, it.q0[i], it.h, it.b);
          tma_store_commit();
        }
        store_pending = true;
      }
    }
    if (row == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

int make_map_bhsd(CUtensorMap* tm, const void* base, int D, int S, int H, int B, const int64_t st[3]) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)H, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)st[2] * 2, (uint64_t)st[1] * 2, (uint64_t)st[0] * 2};
  uint32_t box[4] = {64, (uint32_t)kTile, 1, 1};
  return encode_tmap_16bit(tm, base, 4, dims, strides, box, 1);
}

template <int D, bool BF16, int EMU, bool SPLITP>
int launch_fmha(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv, int Sq, int kv_len,
                const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, float scale, int causal,
                bool persistent, cudaStream_t stream) {
  using L = FmhaSmem<D>;
  using LP = FmhaPSmem<D>;
  auto kfn = fmha_fwd_kernel<D, BF16, EMU, SPLITP>;
  auto kfn_p = fmha_fwd_persistent_kernel<D, BF16, EMU, SPLITP>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal) != cudaSuccess ||
        cudaFuncSetAttribute(kfn_p, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LP::kTotal) != cudaSuccess) {
      (void)cudaGetLastError();
      return B200K_ECUDA;
    }
    configured[dev & 63] = true;
  }
  CUtensorMap tmQ, tmK, tmV, tmO;
  int r;
  if ((r = make_map_bhsd(&tmQ, Q, D, Sq, Hq, B, qs))) return r;
  if ((r = make_map_bhsd(&tmK, K, D, kv_len, Hkv, B, ks))) return r;
  if ((r = make_map_bhsd(&tmV, V, D, kv_len, Hkv, B, vs))) return r;
  if ((r = make_map_bhsd(&tmO, O, D, Sq, Hq, B, os))) return r;
  FmhaParams p;
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sq = Sq;
  p.kv_len = kv_len;
  p.causal = causal;
  p.num_pairs = (Sq + 2 * kTile - 1) / (2 * kTile);
  p.scale_log2 = scale * 1.4426950408889634f;
  // K and V of every (batch, kv head): 2 tensors x 2 bytes
  const double kv_bytes = 4.0 * B * Hkv * (double)kv_len * D;
  p.head_major = kv_bytes > 48.0 * 1024 * 1024 ? 1 : 0;
  p.status = status_ptr();
  if (!p.status) return B200K_ECUDA;
  const long grid = (long)p.num_pairs * Hq * B;
  if (grid <= 0 || grid > 0x7fffffffL) return B200K_ESHAPE;
  // launched so that the set-up may overlap the tail of the kernel before it in the stream (the kernels
  // wait for that kernel before they touch Q, K, V or O); B200K_OPT_PDL = 2 asks for a plain launch
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kFmhaThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning_option(B200K_OPT_PDL) == 2 ? 0 : 1;
  cudaError_t e;
  if (persistent) {
    const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
    cfg.gridDim = dim3((unsigned)(grid < sms ? grid : sms));
    cfg.dynamicSmemBytes = LP::kTotal;
    e = cudaLaunchKernelEx(&cfg, kfn_p, tmQ, tmK, tmV, tmO, p, (int)grid);
  } else {
    cfg.gridDim = dim3((unsigned)grid);
    cfg.dynamicSmemBytes = L::kTotal;
    e = cudaLaunchKernelEx(&cfg, kfn, tmQ, tmK, tmV, tmO, p);
  }
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return B200K_ECUDA;
  }
  return check_launch();
}

bool strides_ok(const void* ptr, const int64_t* st) {
  return aligned16(ptr) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0 && st[0] >= 0 && st[1] >= 0 &&
         st[2] > 0;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_fmha_fwd(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv, int Sq,
                              int Skv, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3], const int64_t o_strides[3], float scale, int causal,
                              int kv_len, int dtype, int variant, b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0) return B200K_ESHAPE;
  if (D != 64 && D != 128) return B200K_EHEADDIM;
  if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides) return B200K_EARG;
  if (kv_len <= 0 || kv_len > Skv) return B200K_EARG;
  if (!(scale > 0.f)) return B200K_EARG;
  if (!strides_ok(Q, q_strides) || !strides_ok(K, k_strides) || !strides_ok(V, v_strides) ||
      !strides_ok(O, o_strides))
    return B200K_EALIGN;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const bool bf16 = dtype == B200K_BF16;
  // variant: 0 = default; 1, 2, 3, 4, 5 = 0, 2, 4, 1, 3 of every 8 score pairs take their exponential
  // on the FMA pipe instead of the MUFU (kept selectable for ablation)
  // 11 .. 15 = the same five with the persistent kernel
  // Default: the persistent kernel for kv_len <= 4096 (measured +3 % at 4096, +10 % at 2048, +19..31 %
  // at 1024, where per-CTA set-up weighs most), the one-item-per-CTA kernel beyond (measured 5-7 %
  // ahead at 8192 / 16384, where the hardware's dynamic CTA scheduling balances better than the static
  // item lists).  B200K_OPT_FMHA_PERSISTENT overrides.
  const int forced = tuning_option(B200K_OPT_FMHA_PERSISTENT);  // 0 library's choice, 1 persistent, 2 one item per CTA
  const bool persistent = variant != 0 ? variant >= 10 : forced ? forced == 1 : kv_len <= 4096;
  static const int kEmuOfCode[5] = {0, 2, 4, 1, 3};
  const int code = (variant % 10) - 1;
  if (variant != 0 && (code < 0 || code > 4 || variant >= 20)) return B200K_EARG;
  // d = 64: P in TMEM columns of its own (the next block's QK^T no longer waits for this block's PV)
  // when B200K_OPT_FMHA_SPLIT_P = 1 asks for it.  Measured on B200 against P over its S columns
  // (bf16, B = 8, 32 heads): -5 % / +1 % at s = 1024 (full / causal), -3 % / +2 % at 2048, -5 % / -10 % at
  // 8192, where it also displaces the row sums on the tensor pipe: the softmax groups no longer wait for
  // S, and the block period does not move, because the two softmax warps that share a scheduler then
  // contend for its issue slots and MUFU instead of taking turns.  Kept selectable, off by default.
  const bool split_p = D == 64 && tuning_option(B200K_OPT_FMHA_SPLIT_P) == 1;
  // measured best: 2 of 8 emulated, except the one-item kernel at d = 64 with its row sums on the tensor
  // pipe (shared S/P columns only), 3 of 8
  const int emu = variant != 0 ? kEmuOfCode[code] : (D == 64 && !persistent && !split_p) ? 3 : kDefaultEmu;
#define B200K_FMHA(DD, BF, EM, SP)                                                                                  \
  launch_fmha<DD, BF, EM, SP>(Q, K, V, O, B, Hq, Hkv, Sq, kv_len, q_strides, k_strides, v_strides, o_strides, scale, \
                              causal, persistent, stream)
#define B200K_FMHA_EMU(DD, BF, SP)                                                                              \
  (emu == 0 ? B200K_FMHA(DD, BF, 0, SP) : emu == 1 ? B200K_FMHA(DD, BF, 1, SP) : emu == 2 ? B200K_FMHA(DD, BF, 2, SP) \
   : emu == 3 ? B200K_FMHA(DD, BF, 3, SP) : B200K_FMHA(DD, BF, 4, SP))
  if (D == 128) return bf16 ? B200K_FMHA_EMU(128, true, false) : B200K_FMHA_EMU(128, false, false);
  if (split_p) return bf16 ? B200K_FMHA_EMU(64, true, true) : B200K_FMHA_EMU(64, false, true);
  return bf16 ? B200K_FMHA_EMU(64, true, false) : B200K_FMHA_EMU(64, false, false);
#undef B200K_FMHA_EMU
#undef B200K_FMHA
}

