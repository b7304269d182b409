/*
 * b200k.h -- C ABI of libb200k.so: hand-written sm_100a kernels behind the
 * reference's two torch-extension packages (gemm_unified, fmha_unified).
 *
 * Plain pointers and sizes only: no torch types cross this boundary.  Every
 * pointer named "device" is a CUDA device pointer owned by the caller; the
 * library never frees caller memory and launches on the stream it is given
 * (0 = the legacy default stream) without synchronising the host.
 *
 * All functions return B200K_OK (0) or a negative B200K_E* code;
 * b200k_strerror() maps a code to text.  A kernel whose bounded device-side
 * wait expired does not trap: it records a status word that
 * b200k_device_status() reads back after the stream was synchronised.
 */
#ifndef B200K_H_
#define B200K_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* opaque stream handle: pass a cudaStream_t (or torch's stream.cuda_stream) */
typedef void* b200k_stream_t;

enum {
  B200K_OK = 0,
  B200K_EDTYPE = -1,     /* dtype is not B200K_F16 / B200K_BF16 */
  B200K_ESHAPE = -2,     /* negative / zero / inconsistent extents */
  B200K_EALIGN = -3,     /* base pointer or leading dimension breaks the 16-byte rule of TMA */
  B200K_EHEADDIM = -4,   /* head_dim other than 64 or 128 */
  B200K_EWORKSPACE = -5, /* workspace missing or too small */
  B200K_ECUDA = -6,      /* a CUDA runtime / driver call failed */
  B200K_ETIMEOUT = -7,   /* a bounded device-side wait expired (see b200k_device_status) */
  B200K_ETMAP = -8,      /* cuTensorMapEncodeTiled refused the operand */
  B200K_EARG = -9,       /* other invalid argument (e.g. causal together with decode) */
  B200K_ENOGPU = -10,    /* no sm_100 device is current */
  B200K_ESCRATCH = -11   /* problem needs more than the library's fixed built-in scratch */
};

enum { B200K_F16 = 0, B200K_BF16 = 1 };

/* GEMM kernel variants (the `variant` argument of b200k_gemm). */
enum {
  B200K_GEMM_AUTO = 0,      /* heuristic: picks one of the below from M, N, K */
  B200K_GEMM_1CTA = 1,      /* 128x256x64 tiles, one CTA per tile, persistent, warp-specialised */
  B200K_GEMM_2CTA = 2,      /* 256x256x64 tiles on a CTA pair (cta_group::2) */
  B200K_GEMM_SKINNY = 3,    /* M <= 128: weight streaming, split-K inside thread-block clusters */
  B200K_GEMM_1CTA_N128 = 4, /* 128x128x64 tiles: more CTAs for small problems */
  B200K_GEMM_GENERIC = 5,   /* CUDA-core kernel without alignment rules (any M, N, K, ld) */
  B200K_GEMM_2CTA_N128 = 6, /* 256x128x64 tiles on a CTA pair: half-size tiles for problems whose
                               256x256 tiles would leave most of the last round of CTA pairs idle
                               (column slabs of a sharded weight); AUTO takes it where
                               rounds x time per tile predicts at least 6 % */
  B200K_GEMM_1CTA_N64 = 7   /* 128x64x64 tiles: twice the CTAs of 128x128 for problems of a few dozen tiles */
};

/*
 * C[M,N] = A[M,K] . B[K,N]; A, B, C row-major with leading dimensions lda,
 * ldb, ldc in ELEMENTS; fp16 or bf16 in and out, fp32 accumulation.
 * Replaces the host launchers `at::Tensor finegemm_N(const at::Tensor& a,
 * const at::Tensor& b)` of the reference
 * (kernels/gemm/pkg/gemm_unified/csrc/semi/gemm_11_nv.cu:175-216,
 *  kernels/gemm/pkg/gemm_unified/csrc/manual/gemm_12_nv.cu:33-103,
 *  kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:23-47), whose
 * contract is a[i*K+k], b[k*N+j], c[i*N+j] (auto/gemm_0.cu:12-20).
 * The tensor-core variants need 16-byte aligned bases and lda, ldb, ldc
 * multiples of 8 elements; AUTO falls back to GENERIC otherwise.
 * No variant needs a workspace today (the split-K partial sums of B200K_GEMM_SKINNY stay in
 * distributed shared memory): `workspace` may be NULL; the arguments are kept so that a
 * future variant can use one without changing the ABI.
 */
int b200k_gemm(const void* A_device, const void* B_device, void* C_device,
               int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
               int dtype, int variant,
               void* workspace_device, size_t workspace_bytes,
               b200k_stream_t stream);

/*
 * The same product, stored to num_dst (1..8) destinations: C_dsts[i] points at the
 * first element of the [M,N] window inside destination i (all with leading dimension
 * ldc).  With the destinations being the full-width C buffers of the GPUs of one
 * node, mapped into this process (CUDA peer / symmetric memory), rank r computes
 * its column slab of a sharded weight and the epilogue writes every finished tile
 * into all ranks' buffers over NVLink with TMA stores while later tiles are still
 * being computed: GEMM and all-gather in one kernel.  The caller synchronises the
 * ranks afterwards (a barrier) before anyone reads C.  Tensor-core variants only
 * (16-byte alignment rules of b200k_gemm apply to every destination).
 * No counterpart in the reference, which has no multi-GPU path.
 */
int b200k_gemm_scatter(const void* A_device, const void* B_device, void* const* C_dsts,
                       int num_dst, int M, int N, int K,
                       int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                       b200k_stream_t stream);

/*
 * GEMM with an epilogue fused into the accumulator drain (tensor-core variants only,
 * alignment rules of b200k_gemm):
 *   B200K_EPI_ADD     C[M,N]   = A.B + R            R: [M,N], leading dimension ldr (residual add)
 *   B200K_EPI_SWIGLU  C[M,N/2] = silu(P[:,2j]) * P[:,2j+1], P = A.B: B holds the gate and up
 *                     projections with interleaved columns (gate_j at 2j, up_j at 2j+1); N % 16 == 0
 * These are the fusions a Llama layer needs around its projections (residual after o_proj and
 * down_proj, SiLU(gate)*up after the merged gate/up projection); the reference applies its
 * GEMMs to no model and fuses nothing (its only fusion is attention itself), so they have no
 * counterpart there.
 */
enum { B200K_EPI_ADD = 1, B200K_EPI_SWIGLU = 2 };
int b200k_gemm_fused(const void* A_device, const void* B_device, void* C_device, const void* R_device,
                     int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                     int dtype, int epilogue, b200k_stream_t stream);

/* Bytes of workspace b200k_gemm needs for (M,N,K,variant); 0 for every current variant. */
size_t b200k_gemm_workspace_bytes(int M, int N, int K, int variant);

/*
 * Fused multi-head attention forward, O = softmax(Q K^T * scale + mask) V,
 * online softmax in fp32, GQA by kv_head = q_head / (Hq / Hkv).
 * Q, O: [B, Hq, Sq, D]; K, V: [B, Hkv, Skv, D] addressed through
 * (batch, head, row) strides in ELEMENTS, the D axis contiguous.  So both the
 * reference's "bhsd" tensors and "bshd" storage are taken without a copy.
 * kv_len (0 < kv_len <= Skv) masks keys j >= kv_len.
 * causal != 0 masks key j for query i when j > i + (kv_len - Sq): the diagonal ends at
 * the last VALID key (bottom-right alignment).  With Sq == kv_len this is the
 * reference's top-left rule `q_idx < k_idx` (semi/fmha_2_nv.cu:177-180); with Sq != kv_len
 * the two differ (the reference would let query i see keys 0..i only).
 * variant: 0 = the library's choice (persistent kernel up to kv_len 4096, one work
 * item per CTA beyond).  For ablation: 1..5 = one item per CTA with 0, 2, 4, 1, 3 of
 * every 8 exponentials computed by a polynomial on the FMA pipe instead of the
 * MUFU; 11..15 = the same five on the persistent kernel.  Other values: B200K_EARG.
 * Replaces `torch::Tensor finefmha_N(Q, K, V, causal, is_decode,
 * decode_length)` of the reference
 * (kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:395-443,
 *  kernels/fmha/pkg/fmha_unified/csrc/manual/fmha_5_nv.cu:135-187).
 */
int b200k_fmha_fwd(const void* Q_device, const void* K_device, const void* V_device,
                   void* O_device,
                   int B, int Hq, int Hkv, int Sq, int Skv, int D,
                   const int64_t q_strides[3], const int64_t k_strides[3],
                   const int64_t v_strides[3], const int64_t o_strides[3],
                   float scale, int causal, int kv_len, int dtype, int variant,
                   b200k_stream_t stream);

/*
 * Decode-shaped attention (few query rows per sequence, normally Sq == 1)
 * with the key/value range of every (batch, kv-head) cut into `num_splits`
 * chunks that run on different CTAs, followed by a reduction kernel that
 * merges the per-chunk (max, sum, partial O) triples in a fixed order.
 * kv_lens_device: int32[B] on the device with the valid length of each
 * sequence, or NULL for Skv everywhere.  num_splits = 0 lets the library
 * choose.  The workspace holds the partial triples
 * (b200k_fmha_decode_workspace_bytes).  With one split per sequence (chosen
 * when the (batch, kv-head) pairs alone fill the GPU, or asked for) the first
 * kernel writes O itself and the workspace, still required, stays untouched.
 * Has the same reference counterpart as b200k_fmha_fwd with is_decode = true
 * (kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_4_nv.cu:240-243,415-417); the
 * per-sequence length vector is an addition, the reference passes one scalar
 * `decode_length` (kernels/fmha/pkg/fmha_unified/ops.py:18).
 */
int b200k_fmha_decode_splitkv(const void* Q_device, const void* K_device,
                              const void* V_device, void* O_device,
                              int B, int Hq, int Hkv, int Sq, int Skv, int D,
                              const int64_t q_strides[3], const int64_t k_strides[3],
                              const int64_t v_strides[3], const int64_t o_strides[3],
                              float scale, const int32_t* kv_lens_device,
                              int num_splits, int dtype,
                              void* workspace_device, size_t workspace_bytes,
                              b200k_stream_t stream);

/*
 * The same decode attention over a PAGED key/value cache: K_pages, V_pages are
 * [num_pages, Hkv, page_size, D] addressed by (page, head, row) element strides,
 * page_size a multiple of 64; logical keys [n*page_size, (n+1)*page_size) of sequence b
 * live in page block_table[b*max_blocks + n] (int32, device).  kv_lens is required.
 * Workspace as b200k_fmha_decode_workspace_bytes(B, Hq, Hkv, Sq, max_blocks*page_size, D,
 * num_splits).  The TMA producer looks the page up per 64-key tile; nothing else differs
 * from b200k_fmha_decode_splitkv, and for the same cache contents and split count the
 * results are bit-identical.  No counterpart in the reference (its KV tensors are dense).
 */
int b200k_fmha_decode_paged(const void* Q_device, const void* K_pages_device, const void* V_pages_device,
                            void* O_device, int B, int Hq, int Hkv, int Sq, int D,
                            int num_pages, int page_size,
                            const int64_t q_strides[3], const int64_t k_page_strides[3],
                            const int64_t v_page_strides[3], const int64_t o_strides[3],
                            float scale, const int32_t* block_table_device, int max_blocks,
                            const int32_t* kv_lens_device, int num_splits, int dtype,
                            void* workspace_device, size_t workspace_bytes, b200k_stream_t stream);

size_t b200k_fmha_decode_workspace_bytes(int B, int Hq, int Hkv, int Sq, int Skv, int D,
                                         int num_splits);

/* The split count b200k_fmha_decode_splitkv uses for num_splits = 0. */
int b200k_fmha_decode_auto_splits(int B, int Hkv, int Skv);

/*
 * b200k_fmha_decode_splitkv for callers that cannot allocate device memory (a
 * server with a memory pool fixed at start-up, a plugin that does not own the
 * process's allocator, a latency-critical loop where cudaMalloc's implicit
 * synchronisation is not acceptable).  Same arguments and result, but there is
 * no workspace argument: the per-split partial results go to a scratch array
 * built into the library image, b200k_fmha_decode_static_scratch_bytes() bytes
 * (16 MiB) on every GPU that loads the library, held until the process exits.
 * The call allocates nothing (no cudaMalloc / cudaFree / allocating library
 * routine).
 *   - Limit: with more than one split, B * Hq * Sq * splits * (D + 2) * 4 bytes must fit
 *     the scratch.  With num_splits = 0 the split count is lowered until it fits (down
 *     to one split, which keeps no partials and always fits); an explicit num_splits > 1
 *     that does not fit returns B200K_ESCRATCH and launches nothing.
 *   - The first call on each device that uses the array looks up its device address
 *     (one cudaGetSymbolAddress with that device current).  Make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array, and it keeps the previous
 *     call's contents.  Nothing needs clearing (every slot that is read was
 *     written by the same call), but two calls that overlap on the GPU (different
 *     streams, or one thread per stream) race on it: serialise them.
 * No counterpart in the reference, which has neither a split over keys nor a
 * workspace.
 */
int b200k_fmha_decode_splitkv_static(const void* Q_device, const void* K_device,
                                     const void* V_device, void* O_device,
                                     int B, int Hq, int Hkv, int Sq, int Skv, int D,
                                     const int64_t q_strides[3], const int64_t k_strides[3],
                                     const int64_t v_strides[3], const int64_t o_strides[3],
                                     float scale, const int32_t* kv_lens_device,
                                     int num_splits, int dtype, b200k_stream_t stream);

/* Size in bytes of the built-in scratch array of b200k_fmha_decode_splitkv_static. */
size_t b200k_fmha_decode_static_scratch_bytes(void);

/* Text for a return code. */
const char* b200k_strerror(int code);

/*
 * Reads (and clears) the device status word of the current device.  Call after
 * the stream was synchronised.  *code_out: 0 or B200K_ETIMEOUT; *detail_out:
 * (kernel id << 24) | (role << 16) | block index of the first CTA that gave up.
 * Synchronises the device.
 */
int b200k_device_status(int* code_out, int* detail_out);

/* Number of kernels this library has launched in this process (all entry points). */
uint64_t b200k_launch_count(void);

/* 1 when the current device is compute capability 10.x, else 0. */
int b200k_device_supported(void);

/*
 * Introspection for tests (no GPU needed): the exact bit patterns the kernels
 * hand to tcgen05.mma.  smem descriptor: 128-byte swizzle, version 1;
 * instruction descriptor: kind::f16, fp32 accumulate, major 0 = K, 1 = MN.
 * The reference has no counterpart (its kernels use WMMA fragments).
 */
/*
 * Tuning overrides for experiments and tests; 0 = the library's own choice (the default).
 * Each option starts from an environment variable of the same name without `OPT_`
 * (B200K_SKINNY_S, ...), read ONCE when the first launch asks; b200k_set_option changes it
 * afterwards and returns the previous value (or B200K_EARG).  No launch reads the environment.
 *   B200K_OPT_SKINNY_S              K-splits (cluster size, 1..8) of the weight-streaming GEMM
 *   B200K_OPT_SKINNY_BN             its slab width, 128 or 256 columns
 *   B200K_OPT_DECODE_HEADS_PER_CTA  h >= 1: decode grid of (split, groups of h KV heads, sequence)
 *   B200K_OPT_FMHA_PERSISTENT       1 = persistent prefill kernel, 2 = one work item per CTA
 *                                   (the environment variable says 1 / 0)
 *   B200K_OPT_SKINNY_PAIR           weight-streaming GEMM, M <= 64: 1 = clusters of three CTAs over two 128-column
 *                                   slabs each wherever that can run (measured slower; never chosen otherwise)
 *   B200K_OPT_PDL                   programmatic dependent launch of the GEMM and prefill kernels.  Default: a
 *                                   kernel may start (barriers, TMEM, tensor-map prefetch) while the kernel before
 *                                   it in the stream is still running and waits for that kernel before it reads
 *                                   an operand or writes an output.  1 = in addition the caller states that the
 *                                   weight of a weight-streaming GEMM (M <= 128) is a constant, not written by the
 *                                   preceding kernel: its first tiles are requested before that wait.  2 = plain
 *                                   launches.
 *   B200K_OPT_FMHA_SPLIT_P          head_dim 64: 1 = P goes to TMEM columns of its own, so that the next
 *                                   block's QK^T is issued ahead of this block's PV product (measured
 *                                   no faster than P over its S columns, the default)
 * The reference's counterpart is the set of template parameters fixed in each launcher
 * (e.g. kernels/gemm/pkg/gemm_unified/csrc/semi/gemm_11_nv.cu:209-213).
 */
enum {
  B200K_OPT_SKINNY_S = 0,
  B200K_OPT_SKINNY_BN = 1,
  B200K_OPT_DECODE_HEADS_PER_CTA = 2,
  B200K_OPT_FMHA_PERSISTENT = 3,
  B200K_OPT_FMHA_SPLIT_P = 4,
  B200K_OPT_SKINNY_PAIR = 5,
  B200K_OPT_PDL = 6,
  B200K_OPT_COUNT = 7
};
int b200k_set_option(int which, int value);

/*
 * Failure-path self test: launches one warp that waits at most limit_ns (<= 100 ms)
 * on a barrier nothing arrives on, records B200K_ETIMEOUT in the device status word
 * (kernel id 15) and returns normally.  Nothing faults or hangs; after it,
 * b200k_device_status() must report the expiry.  No counterpart in the reference.
 */
int b200k_debug_wait_timeout(uint64_t limit_ns, b200k_stream_t stream);

uint64_t b200k_debug_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes);
uint32_t b200k_debug_instr_desc(int dtype, int a_major, int b_major, int M, int N);

#ifdef __cplusplus
}
#endif
#endif /* B200K_H_ */
