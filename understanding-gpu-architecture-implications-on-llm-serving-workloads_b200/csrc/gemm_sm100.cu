// C[M,N] = A[M,K] . B[K,N], row-major, fp16/bf16 in and out, fp32 accumulate.
//
// Tensor-core path (one CTA per 128 x BN output tile, persistent):
//   warp 0      TMA producer: A box 64(K) x 128(M), B boxes 64(N) x 64(K), 128-byte swizzle,
//               STAGES-deep ring guarded by full/empty mbarriers
//   warp 1      MMA issuer: tcgen05.mma kind::f16, M = 128, N = BN, K = 16, A K-major,
//               B MN-major (B is row-major [K,N], so N is the contiguous axis);
//               accumulator double-buffered in TMEM (2 x BN columns)
//   warps 2..5  epilogue: tcgen05.ld -> fp32 -> 16-bit -> swizzled smem -> TMA store,
//               overlapping the next tile's main loop
// Ragged M, N, K edges are handled by TMA: loads outside the tensor read zero,
// stores outside are clipped.
// The same kernel also runs as a CTA pair (cluster of 2, tcgen05 cta_group::2) on 256 x 256
// tiles: each CTA stages its own half of the operands, the leader issues the MMAs for both.
//
// Reference contract: kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:12-20
// (a[i*K+k], b[k*N+j], c[i*N+j]); reference launchers e.g.
// kernels/gemm/pkg/gemm_unified/csrc/semi/gemm_11_nv.cu:175-216.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace b200k {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
// Tile order: groups of `group_n` n-blocks, n fastest inside a group, so the CTAs resident at one
// time share few A row-slabs and few B column-slabs in L2.  Every group walks all of A once: a wider
// group means fewer passes over A (8192 x 4096 x 11008: 16 instead of 8 n-blocks per group cut the
// kernel's DRAM reads from 527 MB to 369 MB, the operands being 154 MB, and measured +1 % cold, +2.6 %
// under the power cap), as long as the group's B columns (group_n x BN x K) stay L2-resident next to
// the A slabs in flight, and as long as a group still spans only about one wave of tiles (M = 2048
// measured 5 % slower with 16).  The host picks 8 or 16 by that rule.
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group_n, int& mb, int& nb) {
  const int per_group = group_n * num_m;
  const int g = t / per_group;
  const int first_n = g * group_n;
  const int gsz = min(group_n, num_n - first_n);
  const int r = t - g * per_group;
  nb = first_n + r % gsz;
  mb = r / gsz;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// CTAS = 1: one CTA per 128 x BN tile.  CTAS = 2: a CTA pair (cluster of 2, cta_group::2) per
// 256 x BN tile; each CTA loads its own 128 rows of A and its own BN/2 columns of B, the pair
// leader issues one M = 256 MMA that reads both CTAs' shared memory and writes 128 accumulator
// rows into each CTA's TMEM, so every B element is staged once per 256 rows instead of per 128.
template <int CTAS, int BN, int STAGES>
struct GemmSmem {
  static constexpr uint32_t kBnLocal = BN / CTAS;  // B columns staged by one CTA
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = kBnLocal * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kStagingBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 buffers x (32 rows x 128 B)
  static constexpr uint32_t kBarOffset = STAGES * kStageBytes + kStagingBytes;
  static constexpr uint32_t kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

// Output tensor maps: normally one.  With several, every finished tile is stored to each of them
// (the same [M,N] window in the C buffers of several GPUs, reached through peer-mapped memory),
// which reassembles a column-sharded product on all ranks from inside the epilogue.
constexpr int kMaxDst = 8;
struct GemmOutMaps {
  CUtensorMap m[kMaxDst];
};

// Epilogues fused into the accumulator drain:
//   kEpiNone    C = A.B
//   kEpiAdd     C = A.B + R               (residual add; R is [M,N] with leading dimension ldr)
//   kEpiSwiglu  C[:, j] = silu(P[:, 2j]) * P[:, 2j+1] with P = A.B: the weight holds the gate and up
//               projections with their columns interleaved, C has N/2 columns
constexpr int kEpiNone = 0, kEpiAdd = 1, kEpiSwiglu = 2;

template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t u, float& lo, float& hi) {
  if constexpr (BF16) {
    lo = __uint_as_float(u << 16);
    hi = __uint_as_float(u & 0xffff0000u);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    lo = __low2float(h);
    hi = __high2float(h);
  }
}
__device__ __forceinline__ float silu_mul(float gate, float up) {
  return __fdividef(gate, 1.f + __expf(-gate)) * up;
}

template <int CTAS, int BN, int STAGES, bool BF16, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ GemmOutMaps tmC, int num_dst, int M, int N, int K, int* status,
               const uint16_t* __restrict__ R, int64_t ldr, int group_n) {
  using L = GemmSmem<CTAS, BN, STAGES>;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr int kTileM = kBM * CTAS;
  constexpr int kKid = CTAS == 1 ? KID_GEMM : KID_GEMM2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CTAS == 1 ? 0u : cluster_ctarank();  // 0 = pair leader
  const int unit = blockIdx.x / CTAS;                       // CTA (or CTA pair) index
  const int num_units = gridDim.x / CTAS;
  const int num_m = (M + kTileM - 1) / kTileM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4 * CTAS);
    }
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    for (int d = 0; d < num_dst; ++d) prefetch_tmap(&tmC.m[d]);
  }
  if (warp == 1) {
    tmem_alloc<CTAS>(tmem_holder, kTmemCols);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  // programmatic dependent launch: the set-up above may have overlapped the tail of the kernel before this
  // one in the stream; no operand is read and no output written before that kernel has finished
  grid_launch_dependents();
  grid_dependency_wait();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = unit; t < num_tiles && ok; t += num_units) {
        int mb, nb;
        tile_coords(t, num_m, num_n, group_n, mb, nb);
        const int row0 = mb * kTileM + (int)rank * kBM;
        const int col0 = nb * BN + (int)rank * (int)L::kBnLocal;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            report_timeout(status, kKid, ROLE_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if constexpr (CTAS == 1) {
            mbar_expect_tx(&full_bar[stage], L::kStageBytes);
            tma_load_2d(sa, &tmA, &full_bar[stage], kb * kBK, row0);
#pragma unroll
            for (int j = 0; j < (int)L::kBnLocal / 64; ++j)
              tma_load_2d(sb + j * (kBK * 128), &tmB, &full_bar[stage], col0 + j * 64, kb * kBK);
          } else {
            // both CTAs' bytes are counted on the leader's barrier, which the MMA thread waits on
            if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
            const uint32_t bar = map_to_cta(&full_bar[stage], 0);
            tma_load_2d_pair(smem_u32(sa), &tmA, bar, kb * kBK, row0);
#pragma unroll
            for (int j = 0; j < (int)L::kBnLocal / 64; ++j)
              tma_load_2d_pair(smem_u32(sb + j * (kBK * 128)), &tmB, bar, col0 + j * 64, kb * kBK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer (pair leader only) -------------------------
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_f16(BF16 ? 1 : 0, /*a K-major*/ 0, /*b MN-major*/ 1, kTileM, BN);
      uint32_t stage = 0, phase = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int t = unit; t < num_tiles && ok; t += num_units, ++it) {
        const uint32_t acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          report_timeout(status, kKid, ROLE_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report_timeout(status, kKid, ROLE_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t b_addr = a_addr + L::kABytes;
          // A: K-major, rows of 128 B, 8-row groups 1024 B apart.
          // B: MN-major, 64 n per 128-B row, 8 k-rows per 1024-B group (stride offset),
          //    next 64-wide n block kBK*128 B further (leading offset).
          const uint64_t adesc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(b_addr, kBK * 128, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advance 16 k: A by 32 B inside the swizzled row, B by 16 rows of 128 B
            umma_ss<CTAS>(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), idesc,
                          (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit<CTAS>(&empty_bar[stage]);
          if constexpr (CTAS == 2) umma_commit_2cta_to(&empty_bar[stage], 1);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          umma_commit<CTAS>(&tmem_full[acc]);
          if constexpr (CTAS == 2) umma_commit_2cta_to(&tmem_full[acc], 1);
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int ew = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t* stg = staging + ew * 8192;
    uint32_t it = 0, chunk_seq = 0;
    bool ok = true;
    for (int t = unit; t < num_tiles && ok; t += num_units, ++it) {
      int mb, nb;
      tile_coords(t, num_m, num_n, group_n, mb, nb);
      const uint32_t acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) {
        if (lane == 0) report_timeout(status, kKid, ROLE_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = mb * kTileM + (int)rank * kBM + ew * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v[32], w[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + acc * BN + c * 64;
        tmem_ld32(taddr, v);
        tmem_ld32(taddr + 32, w);
        tmem_ld_wait();
        // the two staging buffers alternate chunk by chunk ACROSS tiles (a 64-column tile has one chunk)
        uint8_t* buf = stg + (chunk_seq++ & 1) * 4096;
        const int col0 = nb * BN + c * 64;
        if constexpr (EPI == kEpiAdd) {
          // this thread's row of the residual, 64 columns = 8 chunks of 8 elements
          const int grow = row0 + lane;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 r4 = make_uint4(0, 0, 0, 0);
            if (grow < M && col0 + 8 * j < N)
              r4 = *reinterpret_cast<const uint4*>(R + (int64_t)grow * ldr + col0 + 8 * j);
            uint32_t(&dst)[32] = j < 4 ? v : w;
            const int o = (j & 3) * 8;
            float lo, hi;
            unpack2<BF16>(r4.x, lo, hi);
            dst[o + 0] = __float_as_uint(__uint_as_float(dst[o + 0]) + lo);
            dst[o + 1] = __float_as_uint(__uint_as_float(dst[o + 1]) + hi);
            unpack2<BF16>(r4.y, lo, hi);
            dst[o + 2] = __float_as_uint(__uint_as_float(dst[o + 2]) + lo);
            dst[o + 3] = __float_as_uint(__uint_as_float(dst[o + 3]) + hi);
            unpack2<BF16>(r4.z, lo, hi);
            dst[o + 4] = __float_as_uint(__uint_as_float(dst[o + 4]) + lo);
            dst[o + 5] = __float_as_uint(__uint_as_float(dst[o + 5]) + hi);
            unpack2<BF16>(r4.w, lo, hi);
            dst[o + 6] = __float_as_uint(__uint_as_float(dst[o + 6]) + lo);
            dst[o + 7] = __float_as_uint(__uint_as_float(dst[o + 7]) + hi);
          }
        }
        if (lane == 0) tma_store_wait_read<1>();  // the store that last read `buf` has drained
        __syncwarp();
        if constexpr (EPI == kEpiSwiglu) {
          // 64 accumulator columns = 32 (gate, up) pairs -> 32 outputs = 64 bytes per row; rows of
          // 64 bytes under the 64-byte swizzle: 16-byte chunk g of row r sits at g ^ ((r >> 1) & 3)
          uint8_t* rowp = buf + lane * 64;
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            const uint32_t(&src)[32] = g4 < 2 ? v : w;
            const int o = (g4 & 1) * 16;
            uint4 q;
            q.x = pack2<BF16>(silu_mul(__uint_as_float(src[o + 0]), __uint_as_float(src[o + 1])),
                              silu_mul(__uint_as_float(src[o + 2]), __uint_as_float(src[o + 3])));
            q.y = pack2<BF16>(silu_mul(__uint_as_float(src[o + 4]), __uint_as_float(src[o + 5])),
                              silu_mul(__uint_as_float(src[o + 6]), __uint_as_float(src[o + 7])));
            q.z = pack2<BF16>(silu_mul(__uint_as_float(src[o + 8]), __uint_as_float(src[o + 9])),
                              silu_mul(__uint_as_float(src[o + 10]), __uint_as_float(src[o + 11])));
            q.w = pack2<BF16>(silu_mul(__uint_as_float(src[o + 12]), __uint_as_float(src[o + 13])),
                              silu_mul(__uint_as_float(src[o + 14]), __uint_as_float(src[o + 15])));
            *reinterpret_cast<uint4*>(rowp + ((g4 ^ ((lane >> 1) & 3)) << 4)) = q;
          }
          fence_proxy_async_smem();
          __syncwarp();
          // One bulk group per chunk, ALSO for a chunk that lies outside C and stores nothing (an empty
          // group): `tma_store_wait_read<1>` above relies on chunk c - 2, the last user of this staging
          // buffer, being two groups back.  Without the empty groups a tile with two or more trailing
          // chunks outside C let a later chunk overwrite a buffer a pending store was still reading.
          if (lane == 0) {
            if (row0 < M && col0 < N)
              for (int d = 0; d < num_dst; ++d) tma_store_2d(&tmC.m[d], buf, col0 / 2, row0);
            tma_store_commit();
          }
        } else {
          uint8_t* rowp = buf + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 q;
            q.x = pack2<BF16>(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
            q.y = pack2<BF16>(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            q.z = pack2<BF16>(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            q.w = pack2<BF16>(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = q;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 q;
            q.x = pack2<BF16>(__uint_as_float(w[8 * j + 0]), __uint_as_float(w[8 * j + 1]));
            q.y = pack2<BF16>(__uint_as_float(w[8 * j + 2]), __uint_as_float(w[8 * j + 3]));
            q.z = pack2<BF16>(__uint_as_float(w[8 * j + 4]), __uint_as_float(w[8 * j + 5]));
            q.w = pack2<BF16>(__uint_as_float(w[8 * j + 6]), __uint_as_float(w[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = q;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < M && col0 < N) {
              // several destinations (the scatter entry point): the order rotates with the tile and the
              // chunk, so that the CTAs in flight spread their stores over all destinations' links at
              // any moment instead of walking them in step (the caller rotates the list per rank too)
              int d = num_dst > 1 ? (mb + nb + c) % num_dst : 0;
              for (int i = 0; i < num_dst; ++i) {
                tma_store_2d(&tmC.m[d], buf, col0, row0);
                d = d + 1 == num_dst ? 0 : d + 1;
              }
            }
            tma_store_commit();  // always: see the SwiGLU branch above (empty groups keep the count in step)
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 1)
          mbar_arrive(&tmem_empty[acc]);
        else
          mbar_arrive_cluster(&tmem_empty[acc], 0);  // the leader's MMA thread waits for both CTAs
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the leader may still read this CTA's operands until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// CUDA-core kernel without alignment rules (any M, N, K and leading dimensions).
// 64 x 64 tile, 16-deep k slabs in shared memory, 4 x 4 outputs per thread.
// ---------------------------------------------------------------------------
template <bool BF16>
__device__ __forceinline__ float load16(const void* p, int64_t i) {
  if constexpr (BF16)
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  else
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
template <bool BF16>
__device__ __forceinline__ void store16(void* p, int64_t i, float v) {
  if constexpr (BF16)
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

template <bool BF16>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const void* __restrict__ A, const void* __restrict__ B, void* __restrict__ C, int M, int N, int K,
                    int64_t lda, int64_t ldb, int64_t ldc) {
  __shared__ float sA[16][64 + 1];
  __shared__ float sB[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, kk = i & 15;  // A: row r, k kk
      const int gm = m0 + r, gk = k0 + kk;
      sA[kk][r] = (gm < M && gk < K) ? load16<BF16>(A, (int64_t)gm * lda + gk) : 0.f;
      const int kr = i >> 6, c = i & 63;  // B: k kr, col c
      const int gk2 = k0 + kr, gn = n0 + c;
      sB[kr][c] = (gk2 < K && gn < N) ? load16<BF16>(B, (int64_t)gk2 * ldb + gn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn < N) store16<BF16>(C, (int64_t)gm * ldc + gn, acc[i][j]);
    }
  }
}

template <int CTAS, int BN, int STAGES, bool BF16, int EPI = kEpiNone>
int launch_tc(const void* A, const void* B, void* const* Cs, int num_dst, int M, int N, int K, int64_t lda,
              int64_t ldb, int64_t ldc, cudaStream_t stream, const void* R = nullptr, int64_t ldr = 0) {
  using L = GemmSmem<CTAS, BN, STAGES>;
  auto kfn = gemm_tc_kernel<CTAS, BN, STAGES, BF16, EPI>;
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
  CUtensorMap tmA, tmB;
  GemmOutMaps tmC;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {kBK, kBM};
    int r = encode_tmap_16bit(&tmA, A, 2, dims, str, box, 1);
    if (r) return r;
  }
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, kBK};
    int r = encode_tmap_16bit(&tmB, B, 2, dims, str, box, 1);
    if (r) return r;
  }
  for (int d = 0; d < kMaxDst; ++d) {
    // only the destinations in use are encoded (one in every call but the scatter entry point);
    // unused slots repeat the first map so that the parameter block holds no garbage
    if (d >= num_dst) {
      tmC.m[d] = tmC.m[0];
      continue;
    }
    // the SwiGLU epilogue writes N/2 columns, 32 per chunk (64-byte rows, 64-byte swizzle)
    uint64_t dims[2] = {(uint64_t)(EPI == kEpiSwiglu ? N / 2 : N), (uint64_t)M};
    uint64_t str[1] = {(uint64_t)ldc * 2};
    uint32_t box[2] = {EPI == kEpiSwiglu ? 32u : 64u, 32};
    int r = encode_tmap_16bit(&tmC.m[d], Cs[d], 2, dims, str, box, EPI == kEpiSwiglu ? 2 : 1);
    if (r) return r;
  }
  int* status = status_ptr();
  if (!status) return B200K_ECUDA;
  const int num_tiles = ((M + kBM * CTAS - 1) / (kBM * CTAS)) * ((N + BN - 1) / BN);
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const int units = num_tiles < sms / CTAS ? num_tiles : sms / CTAS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * CTAS));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // B200K_OPT_PDL = 2: plain launch
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning_option(B200K_OPT_PDL) == 2 ? 1 : 2;
  // n-blocks per rasterisation group (see tile_coords): 16 when a group is then still about one wave of
  // tiles or less per m-row count (at least 16 rows of tiles) and its B columns take at most 40 MB of L2
  const int num_m = (M + kBM * CTAS - 1) / (kBM * CTAS);
  const int group_n = (num_m >= 16 && 16.0 * BN * K * 2.0 <= 40.0 * 1024 * 1024) ? 16 : 8;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, tmA, tmB, tmC, num_dst, M, N, K, status,
                                     reinterpret_cast<const uint16_t*>(R), ldr, group_n);
  count_launch();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return B200K_ECUDA;
  }
  return check_launch();
}

template <bool BF16>
int launch_generic(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                   cudaStream_t stream) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  gemm_generic_kernel<BF16><<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc);
  count_launch();
  return check_launch();
}

}  // namespace

}  // namespace b200k

using namespace b200k;

// 65..128 rows against a weight of 75 or more 128-column slabs (N >= 9600: the slabs alone nearly fill
// the GPU, no split-K either way): the 128x128 tile kernel is measured 4-5 % ahead of the weight-streaming
// kernel (graph-replayed, bf16, K = 4096: N = 11008 4.79 vs 4.55 TB/s at M = 128, N = 12288 5.09 vs 4.89),
// whose 16 KB activation tile per stage halves the weight bytes it keeps in flight at these row counts.
// On narrower weights, where the streaming kernel's split-K fills the GPU, it is up to 2x behind.
static bool wide_rows_on_tiles(int M, int N) { return M > 64 && (N + 127) / 128 >= 75; }

extern "C" size_t b200k_gemm_workspace_bytes(int M, int N, int K, int variant) {
  (void)M;
  (void)N;
  (void)K;
  (void)variant;
  return 0;
}

// Between the two CTA-pair tile shapes.  The 256 x 256 tile is the faster one per flop (measured 1572 against
// 1437 TFLOP/s on 8192 x 4096 x 11008), but a problem of few tiles ends in a partly filled last round of the
// persistent grid; the 256 x 128 tile halves that loss.  Estimated time = rounds x time per tile (a half-width
// tile takes 0.547 of a full one); the half-width tile is taken where that predicts at least 6 % (measured at
// M = 8192, K = 4096: N = 1408 0.0783 -> 0.0717 ms, N = 1280 0.0816 -> 0.0760 ms; N = 2688, 2816, 5504, 11008
// predicted and measured slower).
static bool half_width_pair_tiles_win(int M, int N, int sms) {
  const long units = sms / 2 > 0 ? sms / 2 : 1;
  const long rows = (M + 255) / 256;
  const long t256 = rows * ((N + 255) / 256), t128 = rows * ((N + 127) / 128);
  const double e256 = (double)((t256 + units - 1) / units);
  const double e128 = (double)((t128 + units - 1) / units) * 0.547;
  return e128 < 0.94 * e256;
}

extern "C" int b200k_gemm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                          int64_t ldc, int dtype, int variant, void* workspace, size_t workspace_bytes,
                          b200k_stream_t stream_) {
  (void)workspace;
  (void)workspace_bytes;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < N || ldc < N) return B200K_ESHAPE;
  if (!A || !B || !C) return B200K_EARG;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const bool tma_ok = aligned16(A) && aligned16(B) && aligned16(C) && lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0;
  if (variant == B200K_GEMM_AUTO) {
    if (!tma_ok) {
      variant = B200K_GEMM_GENERIC;
    } else {
      const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
      const long pair_tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
      const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
      if (M <= 128 && !wide_rows_on_tiles(M, N))
        // weight streaming (split-K inside clusters where the slabs alone do not fill the GPU): measured
        // ahead of the 128-column tiles without split-K on every width from 4096 to 32000 columns for
        // M <= 64 (up to +25 %), within -4 % .. +10 % of them for M = 100..128
        variant = B200K_GEMM_SKINNY;
      else if (M <= 128)
        variant = B200K_GEMM_1CTA_N128;
      else if (pair_tiles >= sms / 2)  // at least one full wave of 256x256 pair tiles
        variant = half_width_pair_tiles_win(M, N, sms) ? B200K_GEMM_2CTA_N128 : B200K_GEMM_2CTA;
      else if (tiles256 >= sms)
        variant = B200K_GEMM_1CTA;
      else {
        // small problems: 128x128 tiles, or 128x64 when even those leave more than half of the SMs idle
        // (1024^3: 64 -> 128 CTAs)
        const long tiles128 = (long)((M + 127) / 128) * ((N + 127) / 128);
        variant = 2 * tiles128 <= sms ? B200K_GEMM_1CTA_N64 : B200K_GEMM_1CTA_N128;
      }
    }
  }
  const bool bf16 = dtype == B200K_BF16;
  switch (variant) {
    case B200K_GEMM_SKINNY:
      if (!tma_ok) return B200K_EALIGN;
      return launch_skinny(A, B, C, M, N, K, lda, ldb, ldc, bf16, stream);
    case B200K_GEMM_1CTA:
      if (!tma_ok) return B200K_EALIGN;
      return bf16 ? launch_tc<1, 256, 4, true>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream)
                  : launch_tc<1, 256, 4, false>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream);
    case B200K_GEMM_2CTA:
      if (!tma_ok) return B200K_EALIGN;
      return bf16 ? launch_tc<2, 256, 6, true>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream)
                  : launch_tc<2, 256, 6, false>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream);
    case B200K_GEMM_2CTA_N128:
      if (!tma_ok) return B200K_EALIGN;
      return bf16 ? launch_tc<2, 128, 8, true>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream)
                  : launch_tc<2, 128, 8, false>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream);
    case B200K_GEMM_1CTA_N64:
      if (!tma_ok) return B200K_EALIGN;
      return bf16 ? launch_tc<1, 64, 8, true>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream)
                  : launch_tc<1, 64, 8, false>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream);
    case B200K_GEMM_1CTA_N128:
      if (!tma_ok) return B200K_EALIGN;
      return bf16 ? launch_tc<1, 128, 6, true>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream)
                  : launch_tc<1, 128, 6, false>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream);
    case B200K_GEMM_GENERIC:
      return bf16 ? launch_generic<true>(A, B, C, M, N, K, lda, ldb, ldc, stream)
                  : launch_generic<false>(A, B, C, M, N, K, lda, ldb, ldc, stream);
    default:
      return B200K_EARG;
  }
}

extern "C" int b200k_gemm_scatter(const void* A, const void* B, void* const* C_dsts, int num_dst, int M, int N, int K,
                                  int64_t lda, int64_t ldb, int64_t ldc, int dtype, b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < N || ldc < N) return B200K_ESHAPE;
  if (!A || !B || !C_dsts || num_dst < 1 || num_dst > kMaxDst) return B200K_EARG;
  if (!aligned16(A) || !aligned16(B) || lda % 8 || ldb % 8 || ldc % 8) return B200K_EALIGN;
  for (int d = 0; d < num_dst; ++d)
    if (!C_dsts[d] || !aligned16(C_dsts[d])) return B200K_EALIGN;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const long pair_tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
  const bool bf16 = dtype == B200K_BF16;
  if (pair_tiles >= sms / 2)
    return bf16 ? launch_tc<2, 256, 6, true>(A, B, C_dsts, num_dst, M, N, K, lda, ldb, ldc, stream)
                : launch_tc<2, 256, 6, false>(A, B, C_dsts, num_dst, M, N, K, lda, ldb, ldc, stream);
  return bf16 ? launch_tc<1, 128, 6, true>(A, B, C_dsts, num_dst, M, N, K, lda, ldb, ldc, stream)
              : launch_tc<1, 128, 6, false>(A, B, C_dsts, num_dst, M, N, K, lda, ldb, ldc, stream);
}

extern "C" int b200k_gemm_fused(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int64_t lda,
                                int64_t ldb, int64_t ldc, int64_t ldr, int dtype, int epilogue,
                                b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (epilogue != B200K_EPI_ADD && epilogue != B200K_EPI_SWIGLU) return B200K_EARG;
  const int n_out = epilogue == B200K_EPI_SWIGLU ? N / 2 : N;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < N || ldc < n_out) return B200K_ESHAPE;
  if (epilogue == B200K_EPI_SWIGLU && N % 16 != 0) return B200K_ESHAPE;  // pairs, and 16-byte output chunks
  if (!A || !B || !C) return B200K_EARG;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || lda % 8 || ldb % 8 || ldc % 8) return B200K_EALIGN;
  if (epilogue == B200K_EPI_ADD) {
    if (!R) return B200K_EARG;
    if (ldr < N) return B200K_ESHAPE;
    if (!aligned16(R) || ldr % 8) return B200K_EALIGN;
  }
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const long pair_tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
  const bool big = pair_tiles >= sms / 2;
  const bool bf16 = dtype == B200K_BF16;
  // decode-shaped calls stream the weight like the plain skinny GEMM (same rule as b200k_gemm's AUTO)
  if (M <= 128 && !wide_rows_on_tiles(M, N))
    return launch_skinny(A, B, C, M, N, K, lda, ldb, ldc, bf16, stream, epilogue, R, ldr);
#define B200K_FUSED(EP)                                                                                       \
  (big ? (bf16 ? launch_tc<2, 256, 6, true, EP>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream, R, ldr)         \
               : launch_tc<2, 256, 6, false, EP>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream, R, ldr))       \
       : (bf16 ? launch_tc<1, 128, 6, true, EP>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream, R, ldr)         \
               : launch_tc<1, 128, 6, false, EP>(A, B, &C, 1, M, N, K, lda, ldb, ldc, stream, R, ldr)))
  return epilogue == B200K_EPI_ADD ? B200K_FUSED(kEpiAdd) : B200K_FUSED(kEpiSwiglu);
#undef B200K_FUSED
}
