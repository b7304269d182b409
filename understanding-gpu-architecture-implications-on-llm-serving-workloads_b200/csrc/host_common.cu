// Host-side helpers: tensor-map encoding, device status word, error strings.
#include "host_common.h"
#include "ptx.cuh"

#include <atomic>
#include <cstdlib>
#include <mutex>

namespace b200k {

namespace {
constexpr int kMaxDevices = 64;

// status word of each device: [0] code, [1] detail, [2..3] spare
__device__ int g_status[4];

std::atomic<uint64_t> g_launches{0};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return (EncodeTiledFn) nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
}  // namespace

namespace {
// Small cache of encoded tensor maps: serving loops call with the same operands over and over,
// and an encode costs about as much as the rest of a launch.  Keyed by everything that enters
// the encoding; a map is a pure function of the key, so a stale entry cannot be wrong.
struct TmapKey {
  const void* base;
  int rank;
  int swizzle;
  uint64_t dims[4];
  uint64_t strides[3];
  uint32_t box[4];
  bool operator==(const TmapKey& o) const {
    if (base != o.base || rank != o.rank || swizzle != o.swizzle) return false;
    for (int i = 0; i < rank; ++i)
      if (dims[i] != o.dims[i] || box[i] != o.box[i] || (i + 1 < rank && strides[i] != o.strides[i])) return false;
    return true;
  }
};
constexpr int kTmapCacheSize = 64;
struct TmapCache {
  TmapKey keys[kTmapCacheSize];
  CUtensorMap maps[kTmapCacheSize];
  bool used[kTmapCacheSize] = {};
  unsigned next = 0;
  std::mutex mu;
};
TmapCache& tmap_cache() {
  static TmapCache c;
  return c;
}
}  // namespace

int encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200K_ECUDA;
  if (rank < 1 || rank > 4) return B200K_ETMAP;
  TmapKey key{};
  key.base = base;
  key.rank = rank;
  key.swizzle = swizzle;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i + 1 < rank) key.strides[i] = strides_bytes[i];
  }
  TmapCache& cache = tmap_cache();
  {
    std::lock_guard<std::mutex> lock(cache.mu);
    for (int i = 0; i < kTmapCacheSize; ++i)
      if (cache.used[i] && cache.keys[i] == key) {
        *out = cache.maps[i];
        return B200K_OK;
      }
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  // BFLOAT16 and FLOAT16 only differ in how an out-of-range fill would be
  // interpreted; both tile 2-byte elements and the fill used here is zero.
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides,
                  gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B
                  : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                 : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return B200K_ETMAP;
  {
    std::lock_guard<std::mutex> lock(cache.mu);
    const unsigned slot = cache.next++ % kTmapCacheSize;
    cache.keys[slot] = key;
    cache.maps[slot] = *out;
    cache.used[slot] = true;
  }
  return B200K_OK;
}

int* status_ptr() {
  static int* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

namespace {
std::atomic<int> g_options[B200K_OPT_COUNT];
std::once_flag g_options_once;
void read_options_from_env() {
  static const char* const names[B200K_OPT_COUNT] = {"B200K_SKINNY_S", "B200K_SKINNY_BN", "B200K_DECODE_HEADS_PER_CTA",
                                                     "B200K_FMHA_PERSISTENT", "B200K_FMHA_SPLIT_P",
                                                     "B200K_SKINNY_PAIR", "B200K_PDL"};
  for (int i = 0; i < B200K_OPT_COUNT; ++i) {
    const char* e = getenv(names[i]);
    int v = e ? atoi(e) : 0;
    // B200K_FMHA_PERSISTENT keeps its historical meaning in the environment (0 = off, 1 = on);
    // the option's values are 0 = library's choice, 1 = persistent kernel, 2 = one item per CTA
    if (i == B200K_OPT_FMHA_PERSISTENT) v = e ? (e[0] == '1' ? 1 : 2) : 0;
    g_options[i].store(v, std::memory_order_relaxed);
  }
}
}  // namespace

int tuning_option(int which) {
  if (which < 0 || which >= B200K_OPT_COUNT) return 0;
  std::call_once(g_options_once, read_options_from_env);
  return g_options[which].load(std::memory_order_relaxed);
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B200K_OK : B200K_ECUDA;
}

const DevInfo& dev_info() {
  static DevInfo infos[kMaxDevices];
  static bool have[kMaxDevices] = {};
  static std::mutex mu;
  static DevInfo none{0, 0, 0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return none;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DevInfo d{};
    cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    infos[dev] = d;
    have[dev] = true;
  }
  return infos[dev];
}

// One warp waits, with a caller-chosen limit, on an mbarrier that nothing ever arrives on, then
// records the expiry in the status word and returns normally: exercises the path every bounded
// wait of the real kernels takes when it gives up, without faulting or hanging anything.
__global__ void wait_probe_kernel(uint64_t limit_ns, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_limit(&bar, 0, limit_ns)) report_timeout(status, KID_WAIT_PROBE, ROLE_PRODUCER);
}

}  // namespace b200k

extern "C" {

int b200k_debug_wait_timeout(uint64_t limit_ns, b200k_stream_t stream) {
  if (!b200k_device_supported()) return B200K_ENOGPU;
  if (limit_ns == 0 || limit_ns > 100000000ull) return B200K_EARG;  // at most 100 ms
  int* status = b200k::status_ptr();
  if (!status) return B200K_ECUDA;
  b200k::wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_ns, status);
  b200k::count_launch();
  return b200k::check_launch();
}

int b200k_set_option(int which, int value) {
  if (which < 0 || which >= B200K_OPT_COUNT || value < 0) return B200K_EARG;
  const int before = b200k::tuning_option(which);  // makes sure the environment has been read first
  b200k::g_options[which].store(value, std::memory_order_relaxed);
  return before;
}

const char* b200k_strerror(int code) {
  switch (code) {
    case B200K_OK: return "ok";
    case B200K_EDTYPE: return "unsupported dtype (expected fp16 or bf16)";
    case B200K_ESHAPE: return "invalid or inconsistent shape";
    case B200K_EALIGN: return "pointer or leading dimension not 16-byte aligned";
    case B200K_EHEADDIM: return "unsupported head_dim (expected 64 or 128)";
    case B200K_EWORKSPACE: return "workspace missing or too small";
    case B200K_ECUDA: return "CUDA call failed";
    case B200K_ETIMEOUT: return "a bounded device-side wait expired";
    case B200K_ETMAP: return "tensor map encoding failed";
    case B200K_EARG: return "invalid argument";
    case B200K_ENOGPU: return "no sm_100 device is current";
    case B200K_ESCRATCH: return "problem does not fit the library's built-in scratch array";
    default: return "unknown b200k error";
  }
}

int b200k_device_status(int* code_out, int* detail_out) {
  int* p = b200k::status_ptr();
  if (!p) return B200K_ECUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return B200K_ECUDA;
  int host[4] = {0, 0, 0, 0};
  if (cudaMemcpy(host, p, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return B200K_ECUDA;
  if (host[0] != 0) {
    if (cudaMemset(p, 0, sizeof(host)) != cudaSuccess) return B200K_ECUDA;
  }
  if (code_out) *code_out = host[0];
  if (detail_out) *detail_out = host[1];
  return B200K_OK;
}

uint64_t b200k_launch_count(void) { return b200k::g_launches.load(std::memory_order_relaxed); }

int b200k_device_supported(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    (void)cudaGetLastError();
    return 0;
  }
  return b200k::dev_info().cc_major == 10 ? 1 : 0;
}

uint64_t b200k_debug_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return b200k::make_smem_desc_sw128(smem_addr, lbo_bytes, sbo_bytes);
}

uint32_t b200k_debug_instr_desc(int dtype, int a_major, int b_major, int M, int N) {
  return b200k::make_idesc_f16(dtype == B200K_BF16 ? 1 : 0, a_major, b_major, M, N);
}

}  // extern "C"
