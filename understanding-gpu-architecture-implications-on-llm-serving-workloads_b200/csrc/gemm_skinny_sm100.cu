// Skinny GEMM (M <= 128 rows of activations against a large weight): bound by streaming the
// weight B[K,N] from HBM once, so the design goal is CTAs and weight bytes in flight, not MMA
// efficiency.
//
//   * Operands are swapped for the tensor core: the 128 weight columns of a slab are the MMA's
//     M rows (A operand, MN-major because B[K,N] is contiguous along N) and the activation rows
//     are the MMA's N columns (B operand, K-major), padded only to MPAD in {16, 32, 64, 128}.
//     A stage is 64 k-rows of the slab (16 or 32 KB of weights: 256 or 512 contiguous bytes of
//     every k-row) plus MPAD*128 bytes of activations, as many stages as fit (up to 8), so small M
//     leaves room for more weight bytes in flight.
//   * One slab of B (128 columns when the slabs fit one wave of CTAs, else 256) per cluster of S CTAs
//     (S in 1..8, 96..128 CTAs in all); CTA r of the cluster streams k-blocks
//     [r*nkb/S, (r+1)*nkb/S): split-K in a cluster.
//   * Roles per CTA (12 warps): thread 0 initialises the barriers and at once issues the first ring of
//     TMA loads, then keeps loading; one MMA thread (tcgen05.mma M = 128, N = MPAD, K = 16, one per
//     128 weight columns and k-step, accumulators D[weight column][activation row] in TMEM); eight
//     warps that drain; two more that only help in the final step.  Draining and reducing are
//     instruction-bound (the streaming loop itself runs at the HBM rate), hence the many warps.
//   * The split-K partials never go to HBM.  CTA r of a cluster owns a share of the slab's columns.
//     Push scheme: every CTA pushes its fp32 partials of a column straight from the accumulators into
//     the owner's receive buffer (remote shared-memory stores, one slot per source CTA), ONE cluster
//     barrier, then every owner sums its S slots locally in rank order 0..S-1 (bit-identical from run
//     to run), converts and stores its part of C; nothing remote is touched after the barrier, so
//     nobody waits at exit.  Where the buffer would cost a stage of the ring that matters more (wide
//     slabs above 16 rows, 128 activation rows): every
//     CTA writes its partial tile to its own drained stage buffers, cluster barrier, owners pull their
//     columns from all S tiles through distributed shared memory, second barrier before exit.  A
//     cluster of one has final accumulators: its draining warps convert and store C themselves.
//   * The same final step carries the fused epilogues of the wide kernels (EPI: 0 none, 1 residual
//     add in fp32 before rounding, 2 SiLU(gate)*up over interleaved column pairs, output N/2 wide),
//     so the o_proj / down_proj / gate-up projections of a decode step stream their weights the
//     same way.
//
// Reference contract: kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:12-20.  The
// reference's tensor-core rungs cannot run these shapes at all (no bounds checks, M % 128
// required: kernels/gemm/pkg/gemm_unified/csrc/semi/gemm_11_nv.cu:179-199).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include "host_common.h"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kSkBK = 64;
// 12 warps: TMA, MMA, 8 that drain the accumulators, and 2 more that only help in the final reduction
// (draining and reducing are instruction-bound: measured 2.8 us of a 19 us kernel with 6 warps)
constexpr int kSkThreads = 384;
constexpr int kSkDrainGroups = 2;  // groups of four draining warps
// BN = weight columns per CTA (256 or 128): BN/128 MMAs of 128 weight columns per k-step, a weight
// tile of BN*64*2 bytes per stage (32 or 16 KB), a partial tile of MPAD*BN floats.

// T = slabs per cluster.  T = 1: one slab per cluster of S CTAs (above).  T = 2 (128-column slabs, push
// scheme only): a cluster of 3 CTAs streams TWO neighbouring slabs, its k-blocks laid end to end and cut
// into three equal ranges (CTA 0: the first two thirds of slab 0; CTA 1: the rest of slab 0 and the first
// third of slab 1, in two accumulators; CTA 2: the rest of slab 1).  For weights whose slabs alone leave a
// third of the SMs idle (N = 11008: 86 slabs) this puts 129 CTAs to work on two thirds of a slab each
// instead of 86 on a whole one.  The 256 columns of the pair are split into three owner slices; a column
// has at most two contributors, which push into slot (rank - first contributor of the column's slab).
template <int MPAD, int BN, int T = 1>
struct SkinnySmem {
  static_assert(T == 1 || (T == 2 && BN == 128 && MPAD <= 64), "two slabs per cluster: narrow slabs, push scheme");
  static constexpr int kSkBN = BN;
  static constexpr uint32_t kSkWBytes = BN * kSkBK * 2;
  static constexpr uint32_t kXBytes = MPAD * kSkBK * 2;  // activation tile of one stage
  static constexpr uint32_t kStageBytes = kSkWBytes + (kXBytes < 1024 ? 1024 : kXBytes);
  // Split-K reduction, push scheme: partials go straight into the owner's receive buffer (one slot per
  // source CTA, MPAD rows of at most BN/S + 3 columns), which must not alias the stage buffers because
  // peers push while this CTA may still be streaming, so it costs ring stages.  Measured against the pull
  // scheme (a tile that reuses the drained stage buffers): narrow slab up to 64 rows +8..10 %, wide slab
  // at 16 rows +3..5 %; wide slab at 32 rows -5 % (the fifth stage goes), 128 rows -5..-17 % (two of six).
  static constexpr bool kPush = (BN == 128 && MPAD <= 64) || (BN == 256 && MPAD <= 16);
  // T = 2: two slots of MPAD rows of ceil(64 chunks / 3 CTAs) * 4 = 88 columns
  static constexpr uint32_t kRecvBytes = !kPush ? 0 : T == 2 ? MPAD * (2 * 88) * 4 : MPAD * (BN + 32) * 4;
  // one CTA per SM: as many stages as fit in ~208 KB next to the receive buffer, at most 6 (8 narrow)
  static constexpr int kMaxStages = BN == 256 ? 6 : 8;
  static constexpr int kFit = (208 * 1024 - kRecvBytes) / kStageBytes;
  static constexpr int kStages = kFit > kMaxStages ? kMaxStages : kFit;
  static constexpr uint32_t kTileBytes = kPush ? 0 : MPAD * kSkBN * 4;  // fp32 partial tile, reuses the stage buffers
  static constexpr uint32_t kRecvOff = kStages * kStageBytes > kTileBytes ? kStages * kStageBytes : kTileBytes;
  static constexpr uint32_t kBarOff = kRecvOff + kRecvBytes;
  static constexpr uint32_t kTotal = kBarOff + 256 + 1024;  // barriers (2 per stage + 1) and the TMEM address, alignment slack
};

__device__ __forceinline__ uint32_t cluster_size_x() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(n));
  return n;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
template <bool BF16>
__device__ __forceinline__ void unpack2s(uint32_t u, float& lo, float& hi) {
  if constexpr (BF16) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&u);
    lo = __low2float(h);
    hi = __high2float(h);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    lo = __low2float(h);
    hi = __high2float(h);
  }
}
// same formula as the wide kernels' SwiGLU epilogue
__device__ __forceinline__ float silu_mul_s(float gate, float up) {
  return __fdividef(gate, 1.f + __expf(-gate)) * up;
}
template <bool BF16>
__device__ __forceinline__ uint16_t pack1s(float x) {
  if constexpr (BF16) {
    const __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<const uint16_t*>(&v);
  } else {
    const __half v = __float2half_rn(x);
    return *reinterpret_cast<const uint16_t*>(&v);
  }
}
template <bool BF16>
__device__ __forceinline__ float unpack1s(uint16_t u) {
  if constexpr (BF16) {
    return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&u));
  } else {
    return __half2float(*reinterpret_cast<const __half*>(&u));
  }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2s(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <int MPAD, bool BF16, int EPI, int BN, int T = 1>
__global__ void __launch_bounds__(kSkThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   uint16_t* __restrict__ C, int64_t ldc, int M, int N, int K, int* status,
                   const uint16_t* __restrict__ R, int64_t ldr, int early_weights) {
  using L = SkinnySmem<MPAD, BN, T>;
  constexpr int kStages = L::kStages;
  constexpr int kSkBN = BN, kSkSub = BN / 128;
  constexpr int kSpan = T * BN;                         // columns a cluster produces
  constexpr uint32_t kSkWBytes = L::kSkWBytes;
  constexpr uint32_t kAccCols = MPAD < 32 ? 32 : MPAD;  // TMEM columns of one accumulator
  constexpr uint32_t kTmemCols = T * kSkSub * kAccCols;  // T = 2: one accumulator per slab this CTA touches
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t S = cluster_size_x();
  const uint32_t rank = cluster_ctarank();
  const int n0 = (blockIdx.x / S) * kSpan;  // first column of the cluster's slab (of its pair of slabs)
  const int num_kb = (K + kSkBK - 1) / kSkBK;
  // This CTA's range of the cluster's k-blocks; with T = 2 the index runs over slab 0's k-blocks and then
  // slab 1's (index / num_kb = slab, index % num_kb = k-block).
  const int kb_begin = (int)((int64_t)rank * (T * num_kb) / S);
  const int kb_end = (int)((int64_t)(rank + 1) * (T * num_kb) / S);
  const int slab_first = T == 1 ? 0 : kb_begin / num_kb;  // slab of this CTA's first accumulator

  // a stage = the weight tile (kSkBN columns x 64 k-rows) and the activation tile (MPAD rows x 64 k); the
  // two halves can be issued apart (the barrier counts the bytes of both)
  auto load_stage_w = [&](int kb, uint32_t stage) {
    uint8_t* sw = smem + stage * L::kStageBytes;
    const int slab = T == 1 ? 0 : kb / num_kb;
    const int k0 = (kb - slab * num_kb) * kSkBK;
    mbar_expect_tx(&full_bar[stage], kSkWBytes + L::kXBytes);
#pragma unroll
    for (int j = 0; j < kSkBN / 64; ++j)
      tma_load_2d(sw + j * (kSkBK * 128), &tmW, &full_bar[stage], n0 + slab * kSkBN + j * 64, k0);
  };
  auto load_stage_x = [&](int kb, uint32_t stage) {
    uint8_t* sx = smem + stage * L::kStageBytes + kSkWBytes;
    const int slab = T == 1 ? 0 : kb / num_kb;
    tma_load_2d(sx, &tmX, &full_bar[stage], (kb - slab * num_kb) * kSkBK, 0);
  };
  auto load_stage = [&](int kb, uint32_t stage) {
    load_stage_w(kb, stage);
    load_stage_x(kb, stage);
  };
  // k-blocks whose loads thread 0 issues right after initialising the barriers, while the TMEM
  // allocation and the CTA-wide sync are still under way (every stage is free at that point)
  const int kb_pre = min(kb_end, kb_begin + kStages);
  if (threadIdx.x == 32) {
    prefetch_tmap(&tmW);
    prefetch_tmap(&tmX);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    fence_mbar_init();
    // Programmatic dependent launch: this kernel may have started while the one before it in the stream
    // is still running, so that its set-up (and the launch gap) hide under that kernel's tail; it waits
    // for that kernel here, before the first byte is requested.  With `early_weights` (the caller states
    // that the weight is a constant of the model, not something the preceding kernel wrote) the WEIGHTS of
    // the first ring are requested before the wait, which also hides the first HBM round trip; the
    // activations may be the previous kernel's output and always come after it.
    if (early_weights)
      for (int kb = kb_begin; kb < kb_pre; ++kb) load_stage_w(kb, (uint32_t)(kb - kb_begin));
    grid_launch_dependents();  // the next kernel of the stream may start its own set-up
    grid_dependency_wait();
    for (int kb = kb_begin; kb < kb_pre; ++kb) {
      if (!early_weights) load_stage_w(kb, (uint32_t)(kb - kb_begin));
      load_stage_x(kb, (uint32_t)(kb - kb_begin));
    }
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_holder, kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_wait();  // every thread that reads R or writes C is ordered behind the previous kernel
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      // the first ring was issued above: continue with the second use of stage 0
      uint32_t stage = 0, phase = 1;
      for (int kb = kb_pre; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
          report_timeout(status, KID_GEMM, ROLE_PRODUCER);
          break;
        }
        load_stage(kb, stage);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // A = weights, MN-major (64 weight columns per 128-byte row, 8 k-rows per 1024-byte group,
      // second 64-column box kSkBK*128 bytes further); B = activations, K-major.
      constexpr uint32_t idesc = make_idesc_f16(BF16 ? 1 : 0, /*a MN-major*/ 1, /*b K-major*/ 0, 128, MPAD);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          report_timeout(status, KID_GEMM, ROLE_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t w_addr = smem_u32(smem + stage * L::kStageBytes);
        const uint64_t xdesc = make_smem_desc_sw128(w_addr + kSkWBytes, 16, 1024);
        // T = 2: the accumulator of the slab this k-block belongs to; it starts afresh at the CTA's first
        // k-block and at the first k-block of a slab
        const int seg = T == 1 ? 0 : kb / num_kb - slab_first;
        const bool fresh = kb == kb_begin || (T == 2 && kb % num_kb == 0);
#pragma unroll
        for (int sub = 0; sub < kSkSub; ++sub) {
          // weight columns [128*sub, 128*sub+128): two 64-column boxes
          const uint64_t wdesc = make_smem_desc_sw128(w_addr + sub * 2 * (kSkBK * 128), kSkBK * 128, 1024);
#pragma unroll
          for (int k = 0; k < kSkBK / 16; ++k)
            umma_ss<1>(tmem_base + (seg * kSkSub + sub) * kAccCols, wdesc + (uint64_t)(k * 128),
                       xdesc + (uint64_t)(k * 2), idesc, (!fresh || k > 0) ? 1u : 0u);
        }
        umma_commit<1>(&empty_bar[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit<1>(tmem_full);
    }
  } else if (warp < 2 + 4 * kSkDrainGroups) {
    // drain TMEM (lane = weight column, TMEM column = activation row): to C directly, to the owners'
    // receive buffers, or to this CTA's fp32 tile [row][kSkBN] (consecutive lanes, consecutive words).
    // Two groups of four warps (a warp reaches the TMEM lanes of quarter warp % 4) take alternate
    // (128-column, row-chunk) pieces.
    const int ew = warp & 3;
    const int grp = (warp - 2) >> 2;
    const bool have = kb_end > kb_begin;
    // Only one lane polls the accumulator barrier during the main loop; the other 255 draining threads
    // park on a hardware named barrier and issue nothing until it opens.  The verdict travels through
    // shared memory.
    volatile uint32_t* verdict = tmem_holder + 1;
    if (warp == 2 && lane == 0) {
      uint32_t good = 1;
      if (have && !mbar_wait(tmem_full, 0)) {
        report_timeout(status, KID_GEMM, ROLE_EPILOGUE);
        good = 0;
      }
      *verdict = good;
    }
    named_barrier_sync(1, 128 * kSkDrainGroups);
    const bool ok = *verdict != 0;
    tc_fence_after();
    float* tile = reinterpret_cast<float*>(smem);
    constexpr int kChunk = MPAD < 32 ? 16 : 32;
    int piece = 0;
    // T = 2: one pass per accumulator (per slab this CTA streamed a part of); a CTA whose range ends
    // inside its first slab has only the first
    const int num_acc = T == 1 ? kSkSub : (have ? (kb_end - 1) / num_kb - slab_first + 1 : 0);
#pragma unroll 1
    for (int sub = 0; sub < num_acc; ++sub) {
      // column inside the cluster's span of kSpan columns
      const int n = (T == 1 ? sub * 128 : (slab_first + sub) * kSkBN) + ew * 32 + lane;
#pragma unroll 1
      for (int cb = 0; cb < MPAD / kChunk; ++cb, ++piece) {
        if (cb * kChunk >= M) break;
        if (piece % kSkDrainGroups != grp) continue;
        uint32_t v[kChunk];
        if (have && ok) {
          const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + sub * kAccCols + cb * kChunk;
          if constexpr (kChunk == 16)
            tmem_ld16(taddr, v);
          else
            tmem_ld32(taddr, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < kChunk; ++e) v[e] = 0u;
        }
        if (L::kPush && S > 1) {
          // Push this CTA's partial of column n into slot `rank` of the receive buffer of the CTA that
          // owns the column's 16-byte chunk: consecutive lanes, consecutive words (plain remote stores).
          const int c = n >> 2;                                          // chunk of 4 columns of the span
          const int owner = ((c + 1) * (int)S - 1) / (kSpan / 4);        // r with c_begin(r) <= c < c_end(r)
          const int c_first = owner * (kSpan / 4) / (int)S;              // first chunk of the owner's slice
          const int wmax = 4 * ((kSpan / 4 + (int)S - 1) / (int)S);      // floats per row of a slot
          // slot: the source's rank (T = 1: every CTA contributes to every column), or its position among
          // the contributors of the column's slab (T = 2: the first one is the first rank whose range ends
          // beyond the slab's first k-block)
          int slot = (int)rank;
          if constexpr (T == 2) {
            const int slab_kb0 = (slab_first + sub) * num_kb;
            int first = 0;
            while ((int)((int64_t)(first + 1) * (T * num_kb) / S) <= slab_kb0) ++first;
            slot = (int)rank - first;
          }
          uint32_t base;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                       : "=r"(base)
                       : "r"(smem_u32(smem + L::kRecvOff)), "r"((uint32_t)owner));
          base += (uint32_t)((slot * MPAD * wmax + (n - 4 * c_first)) * 4);
#pragma unroll
          for (int e = 0; e < kChunk; ++e) {
            const int m = cb * kChunk + e;
            if (m < M)
              asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(base + (uint32_t)(m * wmax * 4)), "r"(v[e]) : "memory");
          }
          continue;
        }
        if (S == 1) {
          // No split-K: the accumulators are final, so they go straight to C.  Lanes 2j and 2j+1 hold
          // neighbouring columns of the same rows; they swap one value per pair of rows, after which
          // the even lane owns both columns of row e and the odd lane both columns of row e+1.
          const int col = (n0 + n) & ~1;
          const bool odd = lane & 1;
#pragma unroll
          for (int e = 0; e < kChunk; e += 2) {
            const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? v[e] : v[e + 1], 1);
            const int m = cb * kChunk + e + (odd ? 1 : 0);
            float lo = __uint_as_float(odd ? got : v[e]);
            float hi = __uint_as_float(odd ? v[e + 1] : got);
            if (m < M && col < N) {
              if constexpr (EPI == 2) {
                C[(int64_t)m * ldc + col / 2] = pack1s<BF16>(silu_mul_s(lo, hi));
              } else if (col + 1 < N) {
                if constexpr (EPI == 1) {
                  float rl, rh;
                  unpack2s<BF16>(*reinterpret_cast<const uint32_t*>(R + (int64_t)m * ldr + col), rl, rh);
                  lo += rl;
                  hi += rh;
                }
                *reinterpret_cast<uint32_t*>(C + (int64_t)m * ldc + col) = pack2s<BF16>(lo, hi);
              } else {
                // odd N: the last column alone (a C that is a column window of a wider tensor must not
                // be written, nor R read, past column N)
                if constexpr (EPI == 1) lo += unpack1s<BF16>(R[(int64_t)m * ldr + col]);
                C[(int64_t)m * ldc + col] = pack1s<BF16>(lo);
              }
            }
          }
          continue;
        }
#pragma unroll
        for (int e = 0; e < kChunk; ++e) {
          const int m = cb * kChunk + e;
          if (m < M) tile[m * kSkBN + n] = __uint_as_float(v[e]);
        }
      }
    }
  }

  // every CTA's partial tile is complete and visible to the cluster (a cluster of one has no peers:
  // a CTA-wide barrier is enough, and nothing needs to wait for anybody at the end)
  tc_fence_before();
  if (S == 1)
    __syncthreads();
  else
    cluster_sync_all();

  if (S > 1) {
    // this CTA's slice of the tile's 16-byte chunks (any S in 1..8 divides them unevenly at most by one)
    const int c_begin = (int)rank * (kSpan / 4) / (int)S;
    const int c_end = ((int)rank + 1) * (kSpan / 4) / (int)S;
    const int w4 = c_end - c_begin;
    // T = 2: how many CTAs contributed to each slab (those whose k-block range meets the slab's)
    int contributors[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
      contributors[t] = 0;
      if constexpr (T == 2) {
        for (int r = 0; r < (int)S; ++r) {
          const int b = (int)((int64_t)r * (T * num_kb) / S), e = (int)((int64_t)(r + 1) * (T * num_kb) / S);
          if (e > b && e > t * num_kb && b < (t + 1) * num_kb) ++contributors[t];
        }
      }
    }
    const uint32_t tile_addr = smem_u32(smem);
    // base address of every peer's tile in rank order (this CTA's own included)
    uint32_t peer[8];
#pragma unroll
    for (uint32_t s = 0; s < 8; ++s)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[s]) : "r"(tile_addr), "r"(s < S ? s : rank));
    // One item = 4 columns of one row; thread t takes items t, t + 384, ... of the slice, walking
    // (row, chunk) incrementally.  The step is instruction-bound, so the code per item is kept short:
    // the first four peers' loads are issued together (clusters of up to 4 are the common case), the
    // rest in a rolled loop; sums always run in rank order (bit-identical from run to run).
    if (w4 > 0) {
      int row = (int)threadIdx.x / w4, c = (int)threadIdx.x % w4;
      const int step_r = kSkThreads / w4, step_c = kSkThreads % w4;
      for (; row < M; row += step_r) {
        const int n = n0 + (c_begin + c) * 4;
        const uint32_t off = (uint32_t)(row * kSkBN + (c_begin + c) * 4) * 4u;  // pull scheme (T = 1) only
        // partial of source CTA s: pushed into this CTA's receive buffer (narrow slab), or read from the
        // source's own tile through distributed shared memory (wide slab)
        auto part = [&](uint32_t s) -> float4 {
          if constexpr (L::kPush) {
            const int wmax = 4 * ((kSpan / 4 + (int)S - 1) / (int)S);
            return *reinterpret_cast<const float4*>(smem + L::kRecvOff +
                                                    (((int)s * MPAD + row) * wmax + c * 4) * 4);
          } else {
            return ld_dsmem_f4(peer[s] + off);
          }
        };
        // sources of this chunk: all S CTAs, or (T = 2) the contributors of the chunk's slab, slots 0..
        const uint32_t nsrc = T == 1 ? S : (uint32_t)contributors[(c_begin + c) / (kSkBN / 4) < T ? (c_begin + c) / (kSkBN / 4) : T - 1];
        float4 acc = nsrc > 0 ? part(0) : make_float4(0.f, 0.f, 0.f, 0.f), v1, v2, v3;
        if (nsrc > 1) v1 = part(1);
        if (nsrc > 2) v2 = part(2);
        if (nsrc > 3) v3 = part(3);
        auto add = [&](const float4& v) {
          acc.x += v.x;
          acc.y += v.y;
          acc.z += v.z;
          acc.w += v.w;
        };
        if (nsrc > 1) add(v1);
        if (nsrc > 2) add(v2);
        if (nsrc > 3) add(v3);
#pragma unroll 1
        for (uint32_t s = 4; s < nsrc; ++s) add(part(s));
        if (n < N) {
          if constexpr (EPI == 2) {
            // columns n..n+3 are (gate, up), (gate, up) of outputs n/2 and n/2+1
            *reinterpret_cast<uint32_t*>(C + (int64_t)row * ldc + n / 2) =
                pack2s<BF16>(silu_mul_s(acc.x, acc.y), silu_mul_s(acc.z, acc.w));
          } else if (n + 3 >= N) {
            // ragged last chunk (N not a multiple of 4): element by element, nothing past column N
            const float part4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (n + e < N) {
                float x = part4[e];
                if constexpr (EPI == 1) x += unpack1s<BF16>(R[(int64_t)row * ldr + n + e]);
                C[(int64_t)row * ldc + n + e] = pack1s<BF16>(x);
              }
            }
          } else {
            if constexpr (EPI == 1) {
              const uint2 r2 = *reinterpret_cast<const uint2*>(R + (int64_t)row * ldr + n);
              float lo, hi;
              unpack2s<BF16>(r2.x, lo, hi);
              acc.x += lo;
              acc.y += hi;
              unpack2s<BF16>(r2.y, lo, hi);
              acc.z += lo;
              acc.w += hi;
            }
            uint2 o;
            o.x = pack2s<BF16>(acc.x, acc.y);
            o.y = pack2s<BF16>(acc.z, acc.w);
            *reinterpret_cast<uint2*>(C + (int64_t)row * ldc + n) = o;
          }
        }
        c += step_c;
        if (c >= w4) {
          c -= w4;
          ++row;
        }
      }
    }
  }

  // pull scheme: nobody leaves while a peer may still read its tile (after the push scheme's single
  // barrier nobody touches another CTA's memory any more)
  if (S > 1 && !L::kPush) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

}  // namespace

// Slab width and cluster size (K-splits per slab).  Measured on B200 (graph-replayed, M = 16..128):
// 128-column slabs beat 256-column ones whenever they fit one wave (N = 4096: +20 %, 11008 x 4096:
// +11..22 %; equal at N = 11008), because the partial tile a CTA has to drain and reduce is half as
// large and fewer K-splits are needed for the same number of CTAs; beyond one wave of 128-column
// slabs the 256-column slab is used.  The rate peaks with 96..128 CTAs (more splits add reduction work
// faster than bytes in flight; more CTAs than SMs means a second wave), so S = round(112 / slabs)
// for 128-column slabs, round(96 / slabs) for 256-column ones, at most 8, never more CTAs than SMs.  B200K_OPT_SKINNY_BN / B200K_OPT_SKINNY_S override both.
int skinny_slab_width(int N) {
  const int forced_bn = tuning_option(B200K_OPT_SKINNY_BN);
  if (forced_bn == 128 || forced_bn == 256) return forced_bn;
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  return (N + 127) / 128 <= sms ? 128 : 256;
}
int skinny_cluster_size(int N, int K, int bn) {
  const int tiles = (N + bn - 1) / bn;
  const int num_kb = (K + kSkBK - 1) / kSkBK;
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const int target = bn == 128 ? 112 : 96;  // CTAs in flight at which the measured rate peaks
  int s = (target + tiles / 2) / tiles;
  if (s > 8) s = 8;
  while (s > 1 && s * tiles > sms) --s;
  if (s > num_kb / 2) s = num_kb / 2;
  if (s < 1) s = 1;
  const int v = tuning_option(B200K_OPT_SKINNY_S);
  if (v >= 1 && v <= 8 && v <= num_kb) s = v;
  return s;
}

template <int MPAD, bool BF16, int EPI, int BN, int T = 1>
static int launch_skinny_t(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                           int64_t ldc, cudaStream_t stream, const void* R, int64_t ldr) {
  using L = SkinnySmem<MPAD, BN, T>;
  constexpr int kSkBN = BN;
  auto kfn = gemm_skinny_kernel<MPAD, BF16, EPI, BN, T>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal) != cudaSuccess) {
      (void)cudaGetLastError();
      return B200K_ECUDA;
    }
    configured[dev & 63] = true;
  }
  CUtensorMap tmX, tmW;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {kSkBK, (uint32_t)MPAD};
    int r = encode_tmap_16bit(&tmX, A, 2, dims, str, box, 1);
    if (r) return r;
  }
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, kSkBK};
    int r = encode_tmap_16bit(&tmW, B, 2, dims, str, box, 1);
    if (r) return r;
  }
  int* status = status_ptr();
  if (!status) return B200K_ECUDA;
  // T = 2: clusters of three CTAs, each over a pair of slabs (an odd last slab is paired with columns
  // beyond N, which load as zeros and store nothing)
  const int S = T == 2 ? 3 : skinny_cluster_size(N, K, kSkBN);
  const int tiles = ((N + kSkBN - 1) / kSkBN + T - 1) / T;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * S));
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch (see the kernel's prologue); B200K_OPT_PDL: 2 = off, 1 = weights are
  // constants and may be requested before the previous kernel has finished
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const int pdl = tuning_option(B200K_OPT_PDL);
  cfg.numAttrs = pdl == 2 ? 1 : 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, tmX, tmW, reinterpret_cast<uint16_t*>(C), ldc, M, N, K, status,
                                     reinterpret_cast<const uint16_t*>(R), ldr, pdl == 1 ? 1 : 0);
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return B200K_ECUDA;
  }
  return check_launch();
}

int launch_skinny(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  bool bf16, cudaStream_t stream, int epilogue, const void* R, int64_t ldr) {
  if (M > 128 || epilogue < 0 || epilogue > 2) return B200K_ESHAPE;
  // tiny M on a wide weight: the epilogue is negligible and 512-byte rows stream a little better
  const bool narrow = skinny_slab_width(N) == 128 && !(M <= 32 && (N + 127) / 128 > 64 && !tuning_option(B200K_OPT_SKINNY_BN));
  // Two slabs per cluster of three CTAs (SkinnySmem's T = 2), meant for weights of 75..98 narrow slabs,
  // where one CTA per slab leaves a third or more of the SMs without weight bytes to stream and two CTAs
  // per slab would not fit one wave.  Measured on B200 (graph-replayed, bf16, K = 4096) it LOSES: N = 11008
  // (129 instead of 86 CTAs) 5.34 -> 4.56 TB/s at M = 1, 4.72 -> 4.04 at M = 64; N = 12288 (144 CTAs) halves,
  // because 48 clusters of three do not all fit the GPCs at once.  86 CTAs already stream at 6.2 TB/s, so
  // what the extra CTAs add to the loop is less than the push, cluster barrier and reduction cost that
  // a cluster of one does not pay.  Kept behind B200K_OPT_SKINNY_PAIR = 1 (tests cover it); never chosen.
  const int slabs128 = (N + 127) / 128, num_kb = (K + kSkBK - 1) / kSkBK;
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const bool pair_can = M <= 64 && num_kb >= 8 && (slabs128 + 1) / 2 * 3 <= sms && slabs128 >= 2 &&
                        tuning_option(B200K_OPT_SKINNY_S) == 0 && tuning_option(B200K_OPT_SKINNY_BN) != 256;
  const int pair_opt = tuning_option(B200K_OPT_SKINNY_PAIR);
  const bool pair = pair_opt == 1 && pair_can;
#define B200K_SKINNY_B(MP, EP, BNN, TT)                                                                      \
  (bf16 ? launch_skinny_t<MP, true, EP, BNN, TT>(A, B, C, M, N, K, lda, ldb, ldc, stream, R, ldr)            \
        : launch_skinny_t<MP, false, EP, BNN, TT>(A, B, C, M, N, K, lda, ldb, ldc, stream, R, ldr))
#define B200K_SKINNY_E(MP, EP) (narrow ? B200K_SKINNY_B(MP, EP, 128, 1) : B200K_SKINNY_B(MP, EP, 256, 1))
#define B200K_SKINNY_P(MP, EP) (pair ? B200K_SKINNY_B(MP, EP, 128, 2) : B200K_SKINNY_E(MP, EP))
#define B200K_SKINNY(MP) \
  return epilogue == 0 ? B200K_SKINNY_P(MP, 0) : epilogue == 1 ? B200K_SKINNY_P(MP, 1) : B200K_SKINNY_P(MP, 2)
  if (M <= 16) { B200K_SKINNY(16); }
  if (M <= 32) { B200K_SKINNY(32); }
  if (M <= 64) { B200K_SKINNY(64); }
#undef B200K_SKINNY_P
#define B200K_SKINNY_P(MP, EP) B200K_SKINNY_E(MP, EP)
  B200K_SKINNY(128);
#undef B200K_SKINNY
#undef B200K_SKINNY_P
#undef B200K_SKINNY_E
#undef B200K_SKINNY_B
}

}  // namespace b200k
