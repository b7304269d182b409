// Compiled torch-op binding of libb200k.so: declares the reference's op schemas and registers CUDA
// implementations that forward to the C ABI (include/b200k.h), with no Python between the
// dispatcher and the kernel launch.
//
// Same shape as the reference's translation units
//   kernels/gemm/pkg/gemm_unified/csrc/gemm_kernel.cu:9-27   TORCH_LIBRARY(gemm_unified, m) { m.def(...) x 17 }
//   kernels/fmha/pkg/fmha_unified/csrc/fmha_kernel.cu:9-18   TORCH_LIBRARY(fmha_unified, m) { m.def(...) x 8 }
// and their per-file TORCH_LIBRARY_IMPL(..., CUDA, m) blocks (e.g. semi/gemm_11_nv.cu:218-220).  Indices
// 0..12 (GEMM) and 0..5 (FMHA) are implemented, 13..16 and 6..7 stay declared only, as in the
// reference's NVIDIA build.  Argument checks mirror the reference launchers' TORCH_CHECKs
// (auto/gemm_0.cu:25-31, semi/fmha_4_nv.cu:397-417) plus bf16 and head_dim 64.
//
// The Python packages load this library when it has been built (gemm_unified/_C.py,
// fmha_unified/_C.py); otherwise they register the same schemas from Python over ctypes.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <cmath>
#include <string>

#include "../../include/b200k.h"

namespace {

int dtype_code(const at::Tensor& t, const char* what) {
  if (t.scalar_type() == at::kHalf) return B200K_F16;
  if (t.scalar_type() == at::kBFloat16) return B200K_BF16;
  TORCH_CHECK(false, what, " must be float16 or bfloat16, got ", t.scalar_type());
  return -1;
}

void check_code(int code, const char* where) {
  TORCH_CHECK(code == 0, where, ": ", b200k_strerror(code), " (code ", code, ")");
}

b200k_stream_t current_stream(const at::Tensor& t) {
  return reinterpret_cast<b200k_stream_t>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

// ------------------------------------------------------------------------------------- GEMM
template <int VARIANT>
at::Tensor finegemm(const at::Tensor& a_in, const at::Tensor& b_in) {
  TORCH_CHECK(a_in.dim() == 2 && b_in.dim() == 2, "a and b must be 2-D");
  TORCH_CHECK(a_in.size(1) == b_in.size(0), "shape mismatch: a is ", a_in.sizes(), ", b is ", b_in.sizes());
  const int dt = dtype_code(a_in, "a and b");
  TORCH_CHECK(b_in.scalar_type() == a_in.scalar_type(), "a and b must have the same dtype");
  TORCH_CHECK(a_in.is_cuda() && b_in.is_cuda(), "a and b must be CUDA tensors");
  TORCH_CHECK(a_in.device() == b_in.device(), "a and b must be on the same device");
  const at::Tensor a = a_in.stride(1) == 1 ? a_in : a_in.contiguous();
  const at::Tensor b = b_in.stride(1) == 1 ? b_in : b_in.contiguous();
  const int64_t M = a.size(0), K = a.size(1), N = b.size(1);
  at::Tensor out = at::empty({M, N}, a.options());
  if (M == 0 || N == 0) return out;
  if (K == 0) return out.zero_();
  const c10::cuda::CUDAGuard guard(a.device());
  check_code(b200k_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                        out.stride(0), dt, VARIANT, nullptr, 0, current_stream(a)),
             "b200k_gemm");
  return out;
}

// ------------------------------------------------------------------------------------- FMHA
constexpr int kDecodeMaxSq = 8;     // decode-shaped calls (few query rows) go to the split-KV kernels
constexpr int kMaxDecodeRows = 16;  // query rows per KV head one split-KV launch takes

void check_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be [batch, heads, seq, head_dim]");
  dtype_code(q, "q, k, v");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(),
              "q, k, v must have the same dtype");
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "q, k, v must be CUDA tensors");
  TORCH_CHECK(q.device() == k.device() && q.device() == v.device(), "q, k, v must be on the same device");
  TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == q.size(0) && k.size(3) == q.size(3), "shape mismatch: q ",
              q.sizes(), ", k ", k.sizes(), ", v ", v.sizes());
  TORCH_CHECK(k.size(1) > 0 && q.size(1) % k.size(1) == 0,
              "number of query heads must be a multiple of the number of KV heads");
  TORCH_CHECK(q.size(3) == 64 || q.size(3) == 128, "head_dim must be 64 or 128, got ", q.size(3));
}

// The kernels need the head_dim axis contiguous and 16-byte aligned strides; anything else (rare) is copied.
at::Tensor rows_contiguous(const at::Tensor& t) {
  if (t.stride(3) != 1 || t.stride(0) % 8 || t.stride(1) % 8 || t.stride(2) % 8 ||
      (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15))
    return t.contiguous();
  return t;
}

struct Strides3 {
  int64_t s[3];
  explicit Strides3(const at::Tensor& t) : s{t.stride(0), t.stride(1), t.stride(2)} {}
};

at::Tensor fmha_fwd(const at::Tensor& q_in, const at::Tensor& k_in, const at::Tensor& v_in, bool causal,
                    int64_t kv_len) {
  const int64_t B = q_in.size(0), Hq = q_in.size(1), Sq = q_in.size(2), D = q_in.size(3);
  const int64_t Hkv = k_in.size(1), Skv = k_in.size(2);
  at::Tensor out = at::empty({B, Hq, Sq, D}, q_in.options());
  if (Sq == 0 || B == 0) return out;
  if (Skv == 0 || kv_len <= 0) return out.zero_();
  const at::Tensor q = rows_contiguous(q_in), k = rows_contiguous(k_in), v = rows_contiguous(v_in);
  const Strides3 qs(q), ks(k), vs(v), os(out);
  const c10::cuda::CUDAGuard guard(q.device());
  check_code(b200k_fmha_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), (int)B, (int)Hq, (int)Hkv,
                            (int)Sq, (int)Skv, (int)D, qs.s, ks.s, vs.s, os.s, 1.0f / std::sqrt((float)D),
                            causal ? 1 : 0, (int)std::min(kv_len, Skv), dtype_code(q, "q"), 0, current_stream(q)),
             "b200k_fmha_fwd");
  return out;
}

// One split-KV launch (at most kMaxDecodeRows query rows per KV head).
void decode_launch(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out,
                   const int32_t* kv_lens) {
  const int64_t B = q.size(0), Hq = q.size(1), Sq = q.size(2), D = q.size(3);
  const int64_t Hkv = k.size(1), Skv = k.size(2);
  const size_t need = b200k_fmha_decode_workspace_bytes((int)B, (int)Hq, (int)Hkv, (int)Sq, (int)Skv, (int)D, 0);
  at::Tensor ws = at::empty({(int64_t)std::max<size_t>(need, 16)}, q.options().dtype(at::kByte));
  const Strides3 qs(q), ks(k), vs(v), os(out);
  check_code(b200k_fmha_decode_splitkv(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), (int)B, (int)Hq,
                                       (int)Hkv, (int)Sq, (int)Skv, (int)D, qs.s, ks.s, vs.s, os.s,
                                       1.0f / std::sqrt((float)D), kv_lens, 0, dtype_code(q, "q"), ws.data_ptr(),
                                       (size_t)ws.numel(), current_stream(q)),
             "b200k_fmha_decode_splitkv");
}

at::Tensor fmha_decode(const at::Tensor& q_in, const at::Tensor& k_in, const at::Tensor& v_in,
                       const c10::optional<at::Tensor>& kv_lens_in) {
  const int64_t B = q_in.size(0), Hq = q_in.size(1), Sq = q_in.size(2), D = q_in.size(3);
  const int64_t Hkv = k_in.size(1), Skv = k_in.size(2);
  at::Tensor out = at::empty({B, Hq, Sq, D}, q_in.options());
  if (Sq == 0 || B == 0) return out;
  if (Skv == 0) return out.zero_();
  const int32_t* lens = nullptr;
  at::Tensor lens_keep;
  if (kv_lens_in.has_value()) {
    const at::Tensor& l = *kv_lens_in;
    TORCH_CHECK(l.scalar_type() == at::kInt && l.device() == q_in.device() && l.numel() == B,
                "kv_lens must be an int32 tensor with one entry per batch element on q's device");
    lens_keep = l.contiguous();
    lens = lens_keep.data_ptr<int32_t>();
  }
  const at::Tensor k = rows_contiguous(k_in), v = rows_contiguous(v_in);
  const c10::cuda::CUDAGuard guard(q_in.device());
  const int64_t group = Hq / Hkv;
  if (group * Sq <= kMaxDecodeRows || Sq > kMaxDecodeRows) {
    const at::Tensor q = rows_contiguous(q_in);
    decode_launch(q, k, v, out, lens);  // Sq > 16 is refused by the library with its own message
    return out;
  }
  // More query rows share a KV head than the kernel's 16-row tile holds (MQA, wide GQA groups): the
  // query heads of every group are taken in slices that fit, each slice one launch over the same K/V.
  int64_t per = 1;
  for (int64_t g = 1; g <= group; ++g)
    if (group % g == 0 && g * Sq <= kMaxDecodeRows) per = g;
  const at::Tensor q5 = q_in.unflatten(1, {Hkv, group});
  at::Tensor o5 = out.unflatten(1, {Hkv, group});
  for (int64_t j = 0; j < group; j += per) {
    const at::Tensor qj = q5.slice(2, j, j + per).flatten(1, 2).contiguous();
    at::Tensor oj = at::empty_like(qj);
    decode_launch(qj, k, v, oj, lens);
    o5.slice(2, j, j + per).copy_(oj.unflatten(1, {Hkv, per}));
  }
  return out;
}

// finefmha_N(q, k, v, causal, is_decode, decode_length): `is_decode` requires !causal
// (semi/fmha_4_nv.cu:415-417) and masks keys beyond decode_length; otherwise decode_length only describes
// padding the reference's Python wrapper added and is applied as the valid key count as well.
at::Tensor finefmha(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool causal, bool is_decode,
                    int64_t decode_length) {
  TORCH_CHECK(!(is_decode && causal), "is_decode and causal cannot be true at the same time");
  check_qkv(q, k, v);
  const int64_t n_kv = k.size(2);
  const int64_t kv_len = decode_length <= 0 ? n_kv : std::min(decode_length, n_kv);
  if (is_decode && q.size(2) <= kDecodeMaxSq) {
    c10::optional<at::Tensor> lens;
    if (kv_len != n_kv) lens = at::full({q.size(0)}, kv_len, q.options().dtype(at::kInt));
    return fmha_decode(q, k, v, lens);
  }
  return fmha_fwd(q, k, v, causal, kv_len);
}

at::Tensor finefmha_decode_varlen(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                  const at::Tensor& kv_lens) {
  check_qkv(q, k, v);
  return fmha_decode(q, k, v, kv_lens);
}

}  // namespace

TORCH_LIBRARY(gemm_unified, m) {
  for (int i = 0; i < 17; ++i)
    m.def(("finegemm_" + std::to_string(i) + "(Tensor a, Tensor b) -> Tensor").c_str());
}

// An index selects a variant of the sm_100a kernel family instead of one of the reference's rungs:
// 0..7, 12 heuristic choice; 8 CUDA-core kernel; 9 128x128 tiles; 10 128x256 tiles; 11 256x256 on a CTA pair.
TORCH_LIBRARY_IMPL(gemm_unified, CUDA, m) {
  m.impl("finegemm_0", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_1", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_2", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_3", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_4", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_5", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_6", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_7", &finegemm<B200K_GEMM_AUTO>);
  m.impl("finegemm_8", &finegemm<B200K_GEMM_GENERIC>);
  m.impl("finegemm_9", &finegemm<B200K_GEMM_1CTA_N128>);
  m.impl("finegemm_10", &finegemm<B200K_GEMM_1CTA>);
  m.impl("finegemm_11", &finegemm<B200K_GEMM_2CTA>);
  m.impl("finegemm_12", &finegemm<B200K_GEMM_AUTO>);
}

TORCH_LIBRARY(fmha_unified, m) {
  for (int i = 0; i < 8; ++i)
    m.def(("finefmha_" + std::to_string(i) +
           "(Tensor q, Tensor k, Tensor v, bool causal, bool is_decode, int decode_length) -> Tensor")
              .c_str());
  // added: a scalar decode_length cannot carry per-sequence KV lengths
  m.def("finefmha_decode_varlen(Tensor q, Tensor k, Tensor v, Tensor kv_lens) -> Tensor");
}

TORCH_LIBRARY_IMPL(fmha_unified, CUDA, m) {
  m.impl("finefmha_0", &finefmha);
  m.impl("finefmha_1", &finefmha);
  m.impl("finefmha_2", &finefmha);
  m.impl("finefmha_3", &finefmha);
  m.impl("finefmha_4", &finefmha);
  m.impl("finefmha_5", &finefmha);
  m.impl("finefmha_decode_varlen", &finefmha_decode_varlen);
}
