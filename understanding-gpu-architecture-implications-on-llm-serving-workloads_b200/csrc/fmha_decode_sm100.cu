// Split-KV attention for decode-shaped inputs (few query rows per sequence).
//
// The workload is bound by HBM: every K and V element is read once and used by the
// (Hq/Hkv * Sq <= 16) query rows that share its KV head, about 4 flop per byte.  So the
// design variable is bytes in flight, not MMA shape:
//   * grid (split, kv head, batch): CTA (s, hk, b) owns keys [s*chunk, (s+1)*chunk) of
//     sequence b, clipped to its valid length kv_lens[b]; CTAs past the length exit.
//   * warp 4 streams 64-key K and V tiles with TMA into a 4-deep ring (128 KB in flight
//     per SM); warps 0-3 each consume a 16-key slice of every tile with ldmatrix +
//     mma.sync m16n8k16 (the query rows padded to the 16-row MMA shape; the tensor-core
//     rate is irrelevant here) and keep their own online-softmax state in registers,
//     row statistics reduced across the 4 lanes of a quad with shuffles.
//   * the 4 warps' states are merged through shared memory in a fixed order and written
//     as one (max, sum, partial O) triple per (row, split) to the fp32 workspace;
//   * a second kernel merges the splits of each row in a fixed order and writes 16-bit O;
//     with one split per sequence the first kernel normalises and writes O itself (same
//     arithmetic, same bits; no partials, no second launch);
//   * unsplit sequences, more (sequence, head) pairs than SMs: the grid is one wave of CTAs
//     and each walks a strided list of pairs; the ring never drains between pairs and the
//     next pair's Q and length are fetched under the current pair's tiles;
//   * the last tile of a sequence is fetched in 16-key slices, only those that hold keys.
// Results are therefore bit-identical from run to run and across work-list shapes.
//
// Reference semantics: is_decode = true of
// kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:240-243,415-417 (non-causal, keys
// beyond the length masked), GQA mapping of semi/fmha_2_nv.cu:36,42-45.  The reference
// pads the single query row to 64 rows (kernels/fmha/pkg/fmha_unified/ops.py:19-25) and
// has no split over keys.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <mutex>

#include "host_common.h"
#include "ptx.cuh"

namespace b200k {
namespace {

constexpr int kDecThreads = 160;  // 4 consumer warps + 1 TMA warp
constexpr int kDecTile = 64;      // keys per stage
constexpr int kDecStages = 4;
constexpr int kMaxRows = 16;

template <int D>
struct DecSmem {
  static constexpr uint32_t kHalfBytes = kDecTile * 128;          // one 64-wide column box
  static constexpr uint32_t kTileBytes = kDecTile * D * 2;        // K or V tile
  static constexpr uint32_t kStageBytes = 2 * kTileBytes;         // K + V
  static constexpr uint32_t kMergeOff = kDecStages * kStageBytes;  // fp32 [4 warps][16 rows][D]
  static constexpr uint32_t kMergeBytes = 4 * kMaxRows * D * 4;
  static constexpr uint32_t kMlOff = kMergeOff + kMergeBytes;      // fp32 [4 warps][16 rows][2]
  // the next item's Q, copied asynchronously under the current item's tiles: 16-bit [2][16 rows][D + 8]
  // (rows 16 bytes apart in the banks: the fragment loads of the 8 row groups do not collide)
  static constexpr uint32_t kQOff = kMlOff + 4 * kMaxRows * 2 * 4;
  static constexpr uint32_t kQRow = D + 8;
  static constexpr uint32_t kBarOff = kQOff + 2 * kMaxRows * kQRow * 2;
  static constexpr uint32_t kTotal = kBarOff + 128 + 1024;
};

struct DecParams {
  const void* q;
  int64_t q_strides[3];
  const int32_t* kv_lens;
  int heads_per_cta;  // consecutive KV heads of one sequence a CTA walks when item_stride == 0
  int item_stride;    // > 0: CTA y walks items y, y + item_stride, ... of the B * Hkv (sequence, head) pairs
  // num_splits == 1: the split kernel normalises and writes O itself (no partials, no second kernel)
  void* out;
  int64_t o_strides[3];
  int out_vec;  // O base 8-byte aligned and strides multiples of 4 elements: 4 columns per store
  float* part_o;   // [B][Hkv][R][num_splits][D]
  float* part_ml;  // [B][Hkv][R][num_splits][2]
  int B, Hq, Hkv, Sq, Skv;
  int rows;        // R = Hq/Hkv * Sq
  int num_splits;
  int chunk;       // keys per split (multiple of kDecTile)
  float scale_log2;
  int* status;
  // paged K/V (block_table == nullptr: one contiguous [B,Hkv,Skv,D] tensor each): the tensor maps
  // then cover [num_pages, Hkv, page_size, D] and logical keys [n*page_size, (n+1)*page_size) of
  // sequence b live in page block_table[b*max_blocks + n]; page_size is a multiple of the 64-key tile
  const int32_t* block_table;
  int max_blocks;
  int page_size;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack_p(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Shared by the kernels below: where row r of a KV head lives in q / o.
__device__ __forceinline__ int64_t row_offset(int r, int hk, int b, int G, int Sq, const int64_t* st) {
  const int head = hk * G + r / Sq;
  const int s = r % Sq;
  return (int64_t)b * st[0] + (int64_t)head * st[1] + (int64_t)s * st[2];
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kDecThreads, 1)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmK16, const __grid_constant__ CUtensorMap tmV16,
                      const DecParams p) {
  using L = DecSmem<D>;
  constexpr int kDBoxes = D / 64;
  constexpr int kDTiles = D / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kDecStages;
  // set by a consumer warp whose wait ran out; read by all four after a barrier so that they leave together
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kDecStages);
  float* merge_o = reinterpret_cast<float*>(smem + L::kMergeOff);
  float* merge_ml = reinterpret_cast<float*>(smem + L::kMlOff);

  // The CTA's work list: items (sequence b, KV head hk) = b * Hkv + hk.
  //   item_stride > 0 (unsplit sequences, one CTA per SM or fewer): items blockIdx.y, + stride, ...
  //   item_stride = 0: heads_per_cta consecutive heads of sequence blockIdx.z
  const int split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_begin = split * p.chunk;
  const int G = p.Hq / p.Hkv;
  int item_first, item_end, item_stride;
  if (p.item_stride > 0) {
    item_first = blockIdx.y;
    item_end = p.B * p.Hkv;
    item_stride = p.item_stride;
  } else {
    const int hk_first = blockIdx.y * p.heads_per_cta;
    item_first = blockIdx.z * p.Hkv + hk_first;
    item_end = blockIdx.z * p.Hkv + min(p.Hkv, hk_first + p.heads_per_cta);
    item_stride = 1;
  }
  auto raw_len = [&](int b) { return p.kv_lens ? p.kv_lens[b] : p.Skv; };
  // tiles of this split in a sequence of (unclamped) length len; k_end = end of its keys
  auto span = [&](int len, int& k_end) {
    len = max(0, min(len, p.Skv));
    k_end = min(len, k_begin + p.chunk);
    return k_begin >= len ? 0 : (k_end - k_begin + kDecTile - 1) / kDecTile;
  };
  // an empty sequence still owns its rows of O in single-split mode: zeros, as the reduction kernel writes
  auto zero_rows = [&](int b, int hk, int tid, int nthreads) {
    for (int i = tid; i < p.rows * D; i += nthreads) {
      const int64_t off = row_offset(i / D, hk, b, G, p.Sq, p.o_strides) + i % D;
      reinterpret_cast<uint16_t*>(p.out)[off] = 0;  // +0 in fp16 and bf16
    }
  };
  if (p.item_stride == 0) {
    // all items share the sequence: a split beyond its length has nothing to do (uniform for the CTA)
    int k_end_unused;
    if (span(raw_len(blockIdx.z), k_end_unused) == 0) {
      if (p.out && split == 0)
        for (int item = item_first; item < item_end; ++item)
          zero_rows(blockIdx.z, item % p.Hkv, threadIdx.x, kDecThreads);
      return;
    }
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmK16);
    prefetch_tmap(&tmV16);
  }
  __syncthreads();

  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      // the length of the next item is asked for one item ahead: its latency must not sit between the
      // last tile of one item and the first of the next
      int cur_len = raw_len(item_first / p.Hkv);
      for (int item = item_first; item < item_end && alive; item += item_stride) {
      const int b = item / p.Hkv, hk = item % p.Hkv;
      const int next_len = item + item_stride < item_end ? raw_len((item + item_stride) / p.Hkv) : 0;
      int k_end;
      const int n_tiles = span(cur_len, k_end);
      cur_len = next_len;
      for (int t = 0; t < n_tiles; ++t) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
          report_timeout(p.status, KID_DECODE, ROLE_PRODUCER);
          alive = false;
          break;
        }
        uint8_t* sk = smem + stage * L::kStageBytes;
        uint8_t* sv = sk + L::kTileBytes;
        int key0 = k_begin + t * kDecTile;
        const int rows_left = k_end - key0;  // >= 1
        int outer = b;
        if (p.block_table) {
          // a 64-key tile never straddles pages; an out-of-range page index makes TMA read zeros
          outer = p.block_table[(int64_t)b * p.max_blocks + key0 / p.page_size];
          key0 %= p.page_size;
        }
        if (rows_left > kDecTile - 16) {
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
#pragma unroll
          for (int d = 0; d < kDBoxes; ++d)
            tma_load_4d(sk + d * L::kHalfBytes, &tmK, &full_bar[stage], d * 64, key0, hk, outer);
#pragma unroll
          for (int d = 0; d < kDBoxes; ++d)
            tma_load_4d(sv + d * L::kHalfBytes, &tmV, &full_bar[stage], d * 64, key0, hk, outer);
        } else {
          // last tile of a sequence with at most 48 keys left: fetch only the 16-key slices that hold
          // keys (same shared-memory image; the slices left alone keep stale data, which the consumers
          // mask in S and zero in V like any key beyond the length)
          const int n16 = (rows_left + 15) / 16;
          mbar_expect_tx(&full_bar[stage], (uint32_t)n16 * 2u * 16u * D * 2u);
          for (int j = 0; j < n16; ++j) {
#pragma unroll
            for (int d = 0; d < kDBoxes; ++d)
              tma_load_4d(sk + d * L::kHalfBytes + j * 16 * 128, &tmK16, &full_bar[stage], d * 64, key0 + 16 * j,
                          hk, outer);
#pragma unroll
            for (int d = 0; d < kDBoxes; ++d)
              tma_load_4d(sv + d * L::kHalfBytes + j * 16 * 128, &tmV16, &full_bar[stage], d * 64, key0 + 16 * j,
                          hk, outer);
          }
        }
        if (++stage == kDecStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      }  // items
    }
  } else {
    // -------------------------------- consumers ---------------------------------
    const int qrow = lane >> 2;  // MMA row of c[0], c[1]; c[2], c[3] are row qrow + 8
    const int qcol = (lane & 3) * 2;
    const float sc = p.scale_log2;
    // ldmatrix lane roles
    const int mi = lane >> 3, mr = lane & 7;
    // the ring's stage and phase run on across the heads this CTA walks
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    // Q as the A operand: 8 k-steps of 16 d; rows >= R are zero.
    auto load_q = [&](int b, int hk, uint32_t (&dst)[D / 16][4]) {
      const uint16_t* qbase = reinterpret_cast<const uint16_t*>(p.q);
      const bool lo_ok = qrow < p.rows, hi_ok = qrow + 8 < p.rows;
      const int64_t off_lo = lo_ok ? row_offset(qrow, hk, b, G, p.Sq, p.q_strides) : 0;
      const int64_t off_hi = hi_ok ? row_offset(qrow + 8, hk, b, G, p.Sq, p.q_strides) : 0;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int d0 = ks * 16 + qcol;
        dst[ks][0] = lo_ok ? *reinterpret_cast<const uint32_t*>(qbase + off_lo + d0) : 0u;
        dst[ks][1] = hi_ok ? *reinterpret_cast<const uint32_t*>(qbase + off_hi + d0) : 0u;
        dst[ks][2] = lo_ok ? *reinterpret_cast<const uint32_t*>(qbase + off_lo + d0 + 8) : 0u;
        dst[ks][3] = hi_ok ? *reinterpret_cast<const uint32_t*>(qbase + off_hi + d0 + 8) : 0u;
      }
    };
    // The following items' Q come through shared memory: a register prefetch is free to be scheduled at
    // its use, and then every item starts with a round trip to HBM (measured: 0.6-0.9 us per item).
    uint16_t* q_stage = reinterpret_cast<uint16_t*>(smem + L::kQOff);
    auto q_copy_async = [&](int b, int hk, int buf) {
      const uint16_t* qbase = reinterpret_cast<const uint16_t*>(p.q);
      for (int i = threadIdx.x; i < p.rows * (D / 2); i += 128) {
        const int r = i / (D / 2), w = i % (D / 2);
        cp_async_4(smem_u32(q_stage + (buf * kMaxRows + r) * L::kQRow + 2 * w),
                   qbase + row_offset(r, hk, b, G, p.Sq, p.q_strides) + 2 * w);
      }
      cp_async_commit();
    };
    auto q_from_stage = [&](int buf, uint32_t (&dst)[D / 16][4]) {
      const bool lo_ok = qrow < p.rows, hi_ok = qrow + 8 < p.rows;
      const uint16_t* lo = q_stage + (buf * kMaxRows + qrow) * L::kQRow;
      const uint16_t* hi = lo + 8 * L::kQRow;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int d0 = ks * 16 + qcol;
        dst[ks][0] = lo_ok ? *reinterpret_cast<const uint32_t*>(lo + d0) : 0u;
        dst[ks][1] = hi_ok ? *reinterpret_cast<const uint32_t*>(hi + d0) : 0u;
        dst[ks][2] = lo_ok ? *reinterpret_cast<const uint32_t*>(lo + d0 + 8) : 0u;
        dst[ks][3] = hi_ok ? *reinterpret_cast<const uint32_t*>(hi + d0 + 8) : 0u;
      }
    };
    int q_buf = 0;
    uint32_t qa[D / 16][4];
    int b = item_first / p.Hkv, hk = item_first % p.Hkv;
    load_q(b, hk, qa);
    int k_end;
    int n_tiles = span(raw_len(b), k_end);
    for (int item = item_first; item < item_end; item += item_stride) {
    // the next item's Q and length are fetched now, under this item's tiles
    const bool has_next = item + item_stride < item_end;
    const int nb = has_next ? (item + item_stride) / p.Hkv : b;
    const int nhk = has_next ? (item + item_stride) % p.Hkv : hk;
    int next_len = 0;
    if (has_next) {
      q_copy_async(nb, nhk, q_buf);
      next_len = raw_len(nb);
    }
    if (n_tiles == 0) {
      if (p.out && split == 0) zero_rows(b, hk, threadIdx.x, 128);
    } else {
    float o[kDTiles][4];
#pragma unroll
    for (int dt = 0; dt < kDTiles; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    for (int t = 0; t < n_tiles; ++t) {
      if (!mbar_wait(&full_bar[stage], phase)) {
        if (lane == 0) {
          report_timeout(p.status, KID_DECODE, ROLE_MMA);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      const uint32_t sk = smem_u32(smem + stage * L::kStageBytes);
      const uint32_t sv = sk + L::kTileBytes;
      const int slice0 = warp * 16;                          // first key of my slice inside the tile
      const int key0 = k_begin + t * kDecTile + slice0;      // its global index
      const int n_valid = k_end - key0;                      // keys of my slice that exist (may be <= 0)
      if (n_valid < 16) {
        // Rows at or beyond the valid length may hold anything (padding of the batch, even
        // NaN): zero them in V so that P = 0 times V stays 0; S is masked below.
        uint8_t* vrow = smem + stage * L::kStageBytes + L::kTileBytes;
#pragma unroll
        for (int it = 0; it < (16 * D * 2 / 16) / 32; ++it) {
          const int cidx = lane + 32 * it;
          const int r = cidx / (D / 8), c16 = cidx % (D / 8);
          if (r >= n_valid)
            *reinterpret_cast<uint4*>(vrow + (c16 >> 3) * L::kHalfBytes + (slice0 + r) * 128 + (c16 & 7) * 16) =
                make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      // ---- S[16 rows x 16 keys] = Q K^T ----
      float sacc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        // matrices: (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
        const int key = slice0 + (mi >> 1) * 8 + mr;
        const int chunk = 2 * ks + (mi & 1);
        const uint32_t addr = sk + (chunk >> 3) * L::kHalfBytes + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(addr, b0, b1, b2, b3);
        mma16816<BF16>(sacc[0], qa[ks], b0, b1);
        mma16816<BF16>(sacc[1], qa[ks], b2, b3);
      }
      // ---- online softmax (rows qrow and qrow + 8; 4 lanes of a quad share a row) ----
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool vis = nt * 8 + qcol + e < n_valid;
          sacc[nt][e] = vis ? sacc[nt][e] * sc : -INFINITY;
          sacc[nt][2 + e] = vis ? sacc[nt][2 + e] * sc : -INFINITY;
          mx_lo = fmaxf(mx_lo, sacc[nt][e]);
          mx_hi = fmaxf(mx_hi, sacc[nt][2 + e]);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float a_lo = (mn_lo == -INFINITY) ? 1.f : ex2f(m_lo - mn_lo);
      const float a_hi = (mn_hi == -INFINITY) ? 1.f : ex2f(m_hi - mn_hi);
      const float sub_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo;
      const float sub_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
      m_lo = mn_lo;
      m_hi = mn_hi;
      uint32_t pa[4];
      float rs_lo = 0.f, rs_hi = 0.f;
      {
        const float p00 = ex2f(sacc[0][0] - sub_lo), p01 = ex2f(sacc[0][1] - sub_lo);
        const float p02 = ex2f(sacc[0][2] - sub_hi), p03 = ex2f(sacc[0][3] - sub_hi);
        const float p10 = ex2f(sacc[1][0] - sub_lo), p11 = ex2f(sacc[1][1] - sub_lo);
        const float p12 = ex2f(sacc[1][2] - sub_hi), p13 = ex2f(sacc[1][3] - sub_hi);
        rs_lo = (p00 + p01) + (p10 + p11);
        rs_hi = (p02 + p03) + (p12 + p13);
        pa[0] = pack_p<BF16>(p00, p01);  // row lo, keys 0-7
        pa[1] = pack_p<BF16>(p02, p03);  // row hi, keys 0-7
        pa[2] = pack_p<BF16>(p10, p11);  // row lo, keys 8-15
        pa[3] = pack_p<BF16>(p12, p13);  // row hi, keys 8-15
      }
      l_lo = l_lo * a_lo + rs_lo;  // per-lane partial sums, reduced across the quad at the end
      l_hi = l_hi * a_hi + rs_hi;
      // ---- O = a * O + P V ----
#pragma unroll
      for (int dp = 0; dp < kDTiles / 2; ++dp) {
        // matrices: (keys 0-7, d tile 2dp), (keys 8-15, 2dp), (keys 0-7, 2dp+1), (keys 8-15, 2dp+1)
        const int key = slice0 + (mi & 1) * 8 + mr;
        const int chunk = 2 * dp + (mi >> 1);
        const uint32_t addr = sv + (chunk >> 3) * L::kHalfBytes + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr, b0, b1, b2, b3);
        float(&oa)[4] = o[2 * dp];
        float(&ob)[4] = o[2 * dp + 1];
        oa[0] *= a_lo; oa[1] *= a_lo; oa[2] *= a_hi; oa[3] *= a_hi;
        ob[0] *= a_lo; ob[1] *= a_lo; ob[2] *= a_hi; ob[3] *= a_hi;
        mma16816<BF16>(oa, pa, b0, b1);
        mma16816<BF16>(ob, pa, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == kDecStages) {
        stage = 0;
        phase ^= 1;
      }
    }
    // a warp whose wait ran out still walks through the barriers below (its partials are garbage and the
    // status word says so); the four warps then stop together
    // ---- quad-reduce the row sums, publish this warp's state ----
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    float* mo = merge_o + warp * kMaxRows * D;
#pragma unroll
    for (int dt = 0; dt < kDTiles; ++dt) {
      // column c of row r sits at c ^ ((r & 3) << 3): the 8 rows of a store spread over the banks
      // (rows beyond the group's are MMA padding: nobody reads them)
      const int pc = (dt * 8 + qcol) ^ ((qrow & 3) << 3);
      if (qrow < p.rows) *reinterpret_cast<float2*>(mo + qrow * D + pc) = make_float2(o[dt][0], o[dt][1]);
      if (qrow + 8 < p.rows)
        *reinterpret_cast<float2*>(mo + (qrow + 8) * D + pc) = make_float2(o[dt][2], o[dt][3]);
    }
    if ((lane & 3) == 0) {
      float* ml = merge_ml + warp * kMaxRows * 2;
      ml[qrow * 2 + 0] = m_lo;
      ml[qrow * 2 + 1] = l_lo;
      ml[(qrow + 8) * 2 + 0] = m_hi;
      ml[(qrow + 8) * 2 + 1] = l_hi;
    }
    named_barrier_sync(1, 128);
    // ---- merge the 4 warps in order 0..3 and write the partial triple ----
    const int tid = threadIdx.x;  // 0..127
    // one item = 4 consecutive columns of one row; GQA groups of up to 4 rows take one pass
    for (int it = tid; it < p.rows * (D / 4); it += 128) {
      const int r = it / (D / 4), c = (it % (D / 4)) * 4;
      float mstar = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mstar = fmaxf(mstar, merge_ml[(w * kMaxRows + r) * 2]);
      float lsum = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const int pc = c ^ ((r & 3) << 3);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = merge_ml[(w * kMaxRows + r) * 2];
        const float wgt = (mw == -INFINITY) ? 0.f : ex2f(mw - mstar);
        lsum += merge_ml[(w * kMaxRows + r) * 2 + 1] * wgt;
        const float4 x = *reinterpret_cast<const float4*>(merge_o + (w * kMaxRows + r) * D + pc);
        acc.x += x.x * wgt;
        acc.y += x.y * wgt;
        acc.z += x.z * wgt;
        acc.w += x.w * wgt;
      }
      if (p.out) {
        // single split: the same arithmetic the reduction kernel does on one partial (weight 2^0 = 1)
        const int64_t off = row_offset(r, hk, b, G, p.Sq, p.o_strides) + c;
        const float v0 = lsum > 0.f ? acc.x / lsum : 0.f, v1 = lsum > 0.f ? acc.y / lsum : 0.f;
        const float v2 = lsum > 0.f ? acc.z / lsum : 0.f, v3 = lsum > 0.f ? acc.w / lsum : 0.f;
        uint16_t* o16 = reinterpret_cast<uint16_t*>(p.out) + off;
        const uint32_t lo = pack_p<BF16>(v0, v1), hi = pack_p<BF16>(v2, v3);
        if (p.out_vec) {
          *reinterpret_cast<uint2*>(o16) = make_uint2(lo, hi);
        } else {
          o16[0] = (uint16_t)lo;
          o16[1] = (uint16_t)(lo >> 16);
          o16[2] = (uint16_t)hi;
          o16[3] = (uint16_t)(hi >> 16);
        }
        continue;
      }
      const int64_t prow = (((int64_t)b * p.Hkv + hk) * p.rows + r) * p.num_splits + split;
      *reinterpret_cast<float4*>(p.part_o + prow * D + c) = acc;
      if (c == 0) {
        p.part_ml[prow * 2 + 0] = mstar;
        p.part_ml[prow * 2 + 1] = lsum;
      }
    }
    }  // item with keys
    if (has_next) {
      // the next item's warps rewrite the merge buffers: everybody must have read them; and everybody's
      // part of the next Q must have landed
      cp_async_wait_all();
      named_barrier_sync(1, 128);
      if (*abort_flag) break;
      q_from_stage(q_buf, qa);
      q_buf ^= 1;
      b = nb;
      hk = nhk;
      n_tiles = span(next_len, k_end);
    }
    }  // items
  }
}

// One CTA per (batch, kv head, row): merges the valid splits in order and writes O.
template <int D, bool BF16>
__global__ void __launch_bounds__(D)
decode_reduce_kernel(const DecParams p, void* __restrict__ out, int64_t os0, int64_t os1, int64_t os2) {
  const int r = blockIdx.x % p.rows;
  const int hk = (blockIdx.x / p.rows) % p.Hkv;
  const int b = blockIdx.x / (p.rows * p.Hkv);
  const int d = threadIdx.x;
  int len = p.kv_lens ? p.kv_lens[b] : p.Skv;
  len = max(0, min(len, p.Skv));
  const int n_valid = len > 0 ? (len + p.chunk - 1) / p.chunk : 0;
  const int64_t prow = (((int64_t)b * p.Hkv + hk) * p.rows + r) * p.num_splits;
  float mstar = -INFINITY;
  for (int s = 0; s < n_valid; ++s) mstar = fmaxf(mstar, p.part_ml[(prow + s) * 2]);
  float lsum = 0.f, acc = 0.f;
  for (int s = 0; s < n_valid; ++s) {
    const float ms = p.part_ml[(prow + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : ex2f(ms - mstar);
    lsum += p.part_ml[(prow + s) * 2 + 1] * w;
    acc += p.part_o[(prow + s) * D + d] * w;
  }
  const float v = lsum > 0.f ? acc / lsum : 0.f;
  const int G = p.Hq / p.Hkv;
  const int64_t st[3] = {os0, os1, os2};
  const int64_t off = row_offset(r, hk, b, G, p.Sq, st) + d;
  if constexpr (BF16)
    reinterpret_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(out)[off] = __float2half_rn(v);
}

// Splits per (batch, KV head).  Measured on B200 (graph-replayed, uniform and ragged lengths): every CTA
// pays about 2-3 us of set-up and pipeline fill, so chunks should be long - about 4096 keys where the
// (batch, head) pairs alone fill the GPU (the 64-sequence ragged batch: 7.0 TB/s with 4-8 splits, 6.7
// with 32) - and where they do not, just enough splits for ONE wave of CTAs (8 sequences x 8 KV heads x
// 8000 keys: 44 us with 2 splits = 128 CTAs, 52-55 us with 3 or 8; one sequence of 32768 keys: 28 us with
// 12-16 splits, 34 us with 37).
int choose_splits(int B, int Hkv, int Skv) {
  const int sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const long pairs = (long)B * Hkv;
  const int by_size = (Skv + 4095) / 4096;
  const int fill = pairs < sms ? (int)(sms / pairs) : 1;
  const int max_by_tile = (Skv + 127) / 128;
  int s = by_size > fill ? by_size : fill;
  if (s > max_by_tile) s = max_by_tile;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

// Work lists of the split kernel's CTAs for unsplit sequences.  Measured on B200 (bf16, d = 128,
// graph-replayed): what decides is how evenly the CTAs fill waves of one per SM and how often a CTA
// pays its set-up (launch, barriers, first round trip to HBM: 2-3 us) - 16 sequences x 32 heads x 4096
// keys: 159 us with 512 CTAs, 152 us with 128 CTAs of 4 heads each; 512 x 8 x 256: 115 us with 4096 or
// 512 CTAs, 107 us with 1024; fewer CTAs than about 0.85 of the SMs loses outright (8 x 32 x 2080 with
// 64 CTAs: 63 us against 44).  So with more (sequence, head) pairs than SMs the grid is one wave of
// CTAs and CTA y walks pairs y, y + G, y + 2G, ... (neighbouring CTAs take the heads of one sequence, a
// CTA's pairs come from sequences spread over the batch, which evens out ragged lengths), with
// G = ceil(pairs / ceil(pairs / SMs)) so that every CTA gets the same count up to one.
int item_stride_of(int B, int Hkv, int splits) {
  if (splits != 1) return 0;
  const long sms = dev_info().sm_count > 0 ? dev_info().sm_count : 148;
  const long pairs = (long)B * Hkv;
  if (pairs <= sms) return 0;
  const long per_cta = (pairs + sms - 1) / sms;
  return (int)((pairs + per_cta - 1) / per_cta);
}

// Override for experiments and tests (B200K_OPT_DECODE_HEADS_PER_CTA): h >= 1 gives the grid
// (split, groups of h consecutive KV heads, sequence) instead, also with split sequences.
int heads_per_cta_override(int Hkv) {
  const int h = tuning_option(B200K_OPT_DECODE_HEADS_PER_CTA);
  if (h < 1) return 0;
  return h < Hkv ? h : Hkv;
}

int chunk_of(int Skv, int splits) {
  const int c = (Skv + splits - 1) / splits;
  return (c + kDecTile - 1) / kDecTile * kDecTile;
}

template <int D, bool BF16>
int launch_decode(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv, int Sq, int Skv,
                  const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, float scale,
                  const int32_t* kv_lens, int splits, float* part_o, float* part_ml, cudaStream_t stream,
                  const int32_t* block_table = nullptr, int max_blocks = 0, int page_size = 0, int num_pages = 0) {
  using L = DecSmem<D>;
  auto kfn = decode_splitkv_kernel<D, BF16>;
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
  CUtensorMap tmK, tmV, tmK16, tmV16;  // 64-key boxes; 16-key boxes for the tail of a sequence
  {
    // contiguous: (D, Skv, Hkv, B); paged: (D, page_size, Hkv, num_pages) with Skv = max_blocks * page_size
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)(block_table ? page_size : Skv), (uint64_t)Hkv,
                        (uint64_t)(block_table ? num_pages : B)};
    uint32_t box[4] = {64, (uint32_t)kDecTile, 1, 1};
    uint64_t kstr[3] = {(uint64_t)ks[2] * 2, (uint64_t)ks[1] * 2, (uint64_t)ks[0] * 2};
    uint64_t vstr[3] = {(uint64_t)vs[2] * 2, (uint64_t)vs[1] * 2, (uint64_t)vs[0] * 2};
    int r;
    if ((r = encode_tmap_16bit(&tmK, K, 4, dims, kstr, box, 1))) return r;
    if ((r = encode_tmap_16bit(&tmV, V, 4, dims, vstr, box, 1))) return r;
    uint32_t box16[4] = {64, 16, 1, 1};
    if ((r = encode_tmap_16bit(&tmK16, K, 4, dims, kstr, box16, 1))) return r;
    if ((r = encode_tmap_16bit(&tmV16, V, 4, dims, vstr, box16, 1))) return r;
  }
  DecParams p;
  p.q = Q;
  p.q_strides[0] = qs[0];
  p.q_strides[1] = qs[1];
  p.q_strides[2] = qs[2];
  p.kv_lens = kv_lens;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.out = splits == 1 ? O : nullptr;
  p.out_vec = (reinterpret_cast<uintptr_t>(O) & 7) == 0 && os[0] % 4 == 0 && os[1] % 4 == 0 && os[2] % 4 == 0;
  p.o_strides[0] = os[0];
  p.o_strides[1] = os[1];
  p.o_strides[2] = os[2];
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sq = Sq;
  p.Skv = Skv;
  p.rows = Hq / Hkv * Sq;
  p.num_splits = splits;
  p.chunk = chunk_of(Skv, splits);
  const int forced = heads_per_cta_override(Hkv);
  p.heads_per_cta = forced ? forced : 1;
  p.item_stride = forced ? 0 : item_stride_of(B, Hkv, splits);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.page_size = page_size;
  p.status = status_ptr();
  if (!p.status) return B200K_ECUDA;
  const dim3 grid = p.item_stride > 0 ? dim3(1, p.item_stride, 1)
                                      : dim3(splits, (Hkv + p.heads_per_cta - 1) / p.heads_per_cta, B);
  kfn<<<grid, kDecThreads, L::kTotal, stream>>>(tmK, tmV, tmK16, tmV16, p);
  count_launch();
  int r = check_launch();
  if (r || splits == 1) return r;
  decode_reduce_kernel<D, BF16><<<B * Hkv * p.rows, D, 0, stream>>>(p, O, os[0], os[1], os[2]);
  count_launch();
  return check_launch();
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200k_fmha_decode_auto_splits(int B, int Hkv, int Skv) {
  if (B <= 0 || Hkv <= 0 || Skv <= 0) return 1;
  return choose_splits(B, Hkv, Skv);
}

extern "C" size_t b200k_fmha_decode_workspace_bytes(int B, int Hq, int Hkv, int Sq, int Skv, int D, int num_splits) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || Hq % Hkv) return 0;
  const int splits = num_splits > 0 ? num_splits : choose_splits(B, Hkv, Skv);
  const size_t rows = (size_t)B * Hkv * (size_t)(Hq / Hkv * Sq);
  return rows * splits * (size_t)(D + 2) * sizeof(float);
}

extern "C" int b200k_fmha_decode_splitkv(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv,
                                         int Sq, int Skv, int D, const int64_t q_strides[3],
                                         const int64_t k_strides[3], const int64_t v_strides[3],
                                         const int64_t o_strides[3], float scale, const int32_t* kv_lens,
                                         int num_splits, int dtype, void* workspace, size_t workspace_bytes,
                                         b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0) return B200K_ESHAPE;
  if (D != 64 && D != 128) return B200K_EHEADDIM;
  if (Hq / Hkv * Sq > kMaxRows) return B200K_ESHAPE;  // more rows per KV head than one MMA tile
  if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides) return B200K_EARG;
  if (!(scale > 0.f) || num_splits < 0 || num_splits > 1024) return B200K_EARG;
  auto ok16 = [](const void* ptr, const int64_t* st) {
    return aligned16(ptr) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
  };
  if (!ok16(K, k_strides) || !ok16(V, v_strides)) return B200K_EALIGN;
  // q is read with 4-byte loads, o written element-wise: even strides suffice for q
  if ((reinterpret_cast<uintptr_t>(Q) & 3) || q_strides[0] % 2 || q_strides[1] % 2 || q_strides[2] % 2)
    return B200K_EALIGN;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const int splits = num_splits > 0 ? num_splits : choose_splits(B, Hkv, Skv);
  const size_t need = b200k_fmha_decode_workspace_bytes(B, Hq, Hkv, Sq, Skv, D, splits);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return B200K_EWORKSPACE;
  const size_t rows = (size_t)B * Hkv * (size_t)(Hq / Hkv * Sq);
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o + rows * splits * D;
  const bool bf16 = dtype == B200K_BF16;
#define B200K_DECODE(DD, BF)                                                                                     \
  launch_decode<DD, BF>(Q, K, V, O, B, Hq, Hkv, Sq, Skv, q_strides, k_strides, v_strides, o_strides, scale, kv_lens, \
                        splits, part_o, part_ml, stream)
  if (D == 128) return bf16 ? B200K_DECODE(128, true) : B200K_DECODE(128, false);
  return bf16 ? B200K_DECODE(64, true) : B200K_DECODE(64, false);
#undef B200K_DECODE
}

extern "C" int b200k_fmha_decode_paged(const void* Q, const void* K_pages, const void* V_pages, void* O, int B, int Hq,
                                       int Hkv, int Sq, int D, int num_pages, int page_size,
                                       const int64_t q_strides[3], const int64_t k_page_strides[3],
                                       const int64_t v_page_strides[3], const int64_t o_strides[3], float scale,
                                       const int32_t* block_table, int max_blocks, const int32_t* kv_lens,
                                       int num_splits, int dtype, void* workspace, size_t workspace_bytes,
                                       b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Hq % Hkv != 0 || num_pages <= 0 || max_blocks <= 0)
    return B200K_ESHAPE;
  if (page_size <= 0 || page_size % kDecTile != 0) return B200K_ESHAPE;
  if ((long)max_blocks * page_size > 0x7fffffffL) return B200K_ESHAPE;
  if (D != 64 && D != 128) return B200K_EHEADDIM;
  if (Hq / Hkv * Sq > kMaxRows) return B200K_ESHAPE;
  if (!Q || !K_pages || !V_pages || !O || !block_table || !kv_lens || !q_strides || !k_page_strides ||
      !v_page_strides || !o_strides)
    return B200K_EARG;
  if (!(scale > 0.f) || num_splits < 0 || num_splits > 1024) return B200K_EARG;
  auto ok16 = [](const void* ptr, const int64_t* st) {
    return aligned16(ptr) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
  };
  if (!ok16(K_pages, k_page_strides) || !ok16(V_pages, v_page_strides)) return B200K_EALIGN;
  if ((reinterpret_cast<uintptr_t>(Q) & 3) || q_strides[0] % 2 || q_strides[1] % 2 || q_strides[2] % 2)
    return B200K_EALIGN;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  const int Skv = max_blocks * page_size;  // logical capacity of a sequence
  const int splits = num_splits > 0 ? num_splits : choose_splits(B, Hkv, Skv);
  const size_t need = b200k_fmha_decode_workspace_bytes(B, Hq, Hkv, Sq, Skv, D, splits);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return B200K_EWORKSPACE;
  const size_t rows = (size_t)B * Hkv * (size_t)(Hq / Hkv * Sq);
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o + rows * splits * D;
  const bool bf16 = dtype == B200K_BF16;
#define B200K_DECODE(DD, BF)                                                                                    \
  launch_decode<DD, BF>(Q, K_pages, V_pages, O, B, Hq, Hkv, Sq, Skv, q_strides, k_page_strides, v_page_strides,  \
                        o_strides, scale, kv_lens, splits, part_o, part_ml, stream, block_table, max_blocks,     \
                        page_size, num_pages)
  if (D == 128) return bf16 ? B200K_DECODE(128, true) : B200K_DECODE(128, false);
  return bf16 ? B200K_DECODE(64, true) : B200K_DECODE(64, false);
#undef B200K_DECODE
}

// ---------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory.
//
// Some hosts of this library must not call cudaMalloc on the path that runs the
// kernel: an inference server whose memory pool was sized at start-up and that
// treats any later driver allocation as a fault, a plugin loaded into a process
// whose allocator it does not own, or code running between the steps of a
// latency-critical loop where an allocation (which may synchronise the device)
// is not acceptable.  For them the split-KV partial results live in the
// file-scope array below instead of a caller-provided workspace.
//
// The array is part of the library image: every GPU that loads libb200k.so holds
// kStaticScratchBytes of its memory until the process exits, whether or not this
// entry point is ever called.  That is why its size is fixed and modest.
// ---------------------------------------------------------------------------
namespace b200k {
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB per GPU

static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// Device address of g_decode_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could
// use, so the address is asked for once per device, with that device current.
int static_scratch_ptr(unsigned char** out) {
  constexpr int kMaxDev = 64;
  static unsigned char* ptrs[kMaxDev] = {};
  static std::mutex mu;  // the per-device table is filled lazily by whichever host thread comes first
  std::lock_guard<std::mutex> lock(mu);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    (void)cudaGetLastError();
    return B200K_ECUDA;
  }
  if (!ptrs[dev]) {
    unsigned char* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_scratch) != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return B200K_ECUDA;
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return B200K_OK;
}

size_t decode_partials_bytes(int B, int Hq, int Hkv, int Sq, int D, int splits) {
  const size_t rows = (size_t)B * Hkv * (size_t)(Hq / Hkv * Sq);
  return rows * (size_t)splits * (size_t)(D + 2) * sizeof(float);
}

}  // namespace
}  // namespace b200k

extern "C" size_t b200k_fmha_decode_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int b200k_fmha_decode_splitkv_static(const void* Q, const void* K, const void* V, void* O, int B, int Hq,
                                                int Hkv, int Sq, int Skv, int D, const int64_t q_strides[3],
                                                const int64_t k_strides[3], const int64_t v_strides[3],
                                                const int64_t o_strides[3], float scale, const int32_t* kv_lens,
                                                int num_splits, int dtype, b200k_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype != B200K_F16 && dtype != B200K_BF16) return B200K_EDTYPE;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0) return B200K_ESHAPE;
  if (D != 64 && D != 128) return B200K_EHEADDIM;
  if (Hq / Hkv * Sq > kMaxRows) return B200K_ESHAPE;
  if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides) return B200K_EARG;
  if (!(scale > 0.f) || num_splits < 0 || num_splits > 1024) return B200K_EARG;
  auto ok16 = [](const void* ptr, const int64_t* st) {
    return aligned16(ptr) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
  };
  if (!ok16(K, k_strides) || !ok16(V, v_strides)) return B200K_EALIGN;
  if ((reinterpret_cast<uintptr_t>(Q) & 3) || q_strides[0] % 2 || q_strides[1] % 2 || q_strides[2] % 2)
    return B200K_EALIGN;
  if (!b200k_device_supported()) return B200K_ENOGPU;
  // An explicit split count must fit the fixed scratch; with 0 the library's usual choice is
  // lowered until it fits.  A problem that does not fit even unsplit is refused.
  int splits = num_splits;
  if (splits == 0) {
    splits = choose_splits(B, Hkv, Skv);
    while (splits > 1 && decode_partials_bytes(B, Hq, Hkv, Sq, D, splits) > kStaticScratchBytes) --splits;
  }
  // One split per sequence keeps no partials at all (the split kernel normalises and writes O itself),
  // so such a call neither has to fit the array nor needs its address.
  unsigned char* scratch = nullptr;
  if (splits > 1) {
    if (decode_partials_bytes(B, Hq, Hkv, Sq, D, splits) > kStaticScratchBytes) return B200K_ESCRATCH;
    int r = static_scratch_ptr(&scratch);
    if (r) return r;
  }
  const size_t rows = (size_t)B * Hkv * (size_t)(Hq / Hkv * Sq);
  // Nothing has to start at zero: every (max, sum, partial O) slot the reduction kernel
  // reads was written by the split kernel of this same call; slots of splits past a
  // sequence's length are neither written nor read.
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o + rows * splits * D;
  const bool bf16 = dtype == B200K_BF16;
#define B200K_DECODE(DD, BF)                                                                                     \
  launch_decode<DD, BF>(Q, K, V, O, B, Hq, Hkv, Sq, Skv, q_strides, k_strides, v_strides, o_strides, scale, kv_lens, \
                        splits, part_o, part_ml, stream)
  if (D == 128) return bf16 ? B200K_DECODE(128, true) : B200K_DECODE(128, false);
  return bf16 ? B200K_DECODE(64, true) : B200K_DECODE(64, false);
#undef B200K_DECODE
}
