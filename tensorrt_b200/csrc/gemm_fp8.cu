// FP8 E4M3 x E4M3 GEMM entry point (tcgen05 kind::f8f6f4) and the pieces shared by both
// quantized GEMMs: the TMA descriptor encoder lookup and the device status word.
#include <cstdlib>
#include <mutex>

#include "gemm_host.cuh"

namespace b200q {
namespace gemm {

namespace {
__device__ int g_device_status = 0;
std::mutex g_mu;
int* g_status_addr[64] = {};
}  // namespace

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    g_status_addr[dev] = static_cast<int*>(p);
  }
  return g_status_addr[dev];
}

bool valid_tile_n(int bn) {
  return bn == 0 || bn == 128 || bn == 256 || bn == 512 || bn == 1001 || bn == 1002 || bn == 1004 || bn == 1008;
}

int sf_copier_enabled() {
  static const int v = [] {
    const char* e = std::getenv("B200Q_SF_COPIER");   // measured 3-4 % faster with the copier warp: on unless set to 0
    return e != nullptr ? std::atoi(e) : 1;
  }();
  return v;
}

int forced_smallm_stages() {
  static const int v = [] {
    const char* e = std::getenv("B200Q_SMALLM_STAGES");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  return v;
}

}  // namespace gemm
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_device_status(int reset) {
  int* w = gemm::device_status_word();
  if (w == nullptr) return B200Q_ERR_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return B200Q_ERR_CUDA;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return B200Q_ERR_CUDA;
  }
  return v == 0 ? B200Q_OK : B200Q_ERR_TIMEOUT;
}

int b200q_fp8_gemm(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel, const uint8_t* b_codes,
                   const float* b_scales, int64_t b_scales_numel, const void* bias, void* out, int64_t M, int64_t N,
                   int64_t K, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || out == nullptr)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && (!gemm::valid_tile_n(cfg->tile_n) || cfg->reserved != 0)) return B200Q_ERR_INVALID;
  if (M < 0 || N < 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 16 != 0) return B200Q_ERR_INVALID;
  if ((a_scales_numel != 1 && a_scales_numel != M) || (b_scales_numel != 1 && b_scales_numel != N)) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (M == 0 || N == 0) return B200Q_OK;
  gemm::Params p{};
  p.a_scales = a_scales;
  p.b_scales = b_scales;
  p.a_scale_stride = a_scales_numel == 1 ? 0 : 1;
  p.b_scale_stride = b_scales_numel == 1 ? 0 : 1;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K);
  return gemm::launch<false>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream), cfg);
}

int b200q_fp8_gemm_silu_mul(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel, const uint8_t* b_codes,
                            const float* b_scales, int64_t b_scales_numel, const void* bias, void* out, int64_t M, int64_t N,
                            int64_t K, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || out == nullptr)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && (cfg->tile_n != 0 || cfg->reserved != 0)) return B200Q_ERR_INVALID;   // one kernel serves this entry
  if (M < 0 || N < 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 16 != 0 || N % 256 != 0) return B200Q_ERR_INVALID;                                   // F = N / 2 in whole 128-column tiles
  if ((a_scales_numel != 1 && a_scales_numel != M) || (b_scales_numel != 1 && b_scales_numel != N)) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (M == 0 || N == 0) return B200Q_OK;
  gemm::Params p{};
  p.a_scales = a_scales;
  p.b_scales = b_scales;
  p.a_scale_stride = a_scales_numel == 1 ? 0 : 1;
  p.b_scale_stride = b_scales_numel == 1 ? 0 : 1;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K);
  p.silu_f = static_cast<int>(N / 2);
  p.status = gemm::device_status_word();
  if (p.status == nullptr) return B200Q_ERR_CUDA;
  return gemm::launch_pair<false, 1>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream));
}

int b200q_fp8_gemm_silu_mul_quantize(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel, const uint8_t* b_codes,
                                     const float* b_scales, int64_t b_scales_numel, const void* bias, const float* act_amax,
                                     uint8_t* codes_out, float* scale_out, int64_t M, int64_t N, int64_t K, b200q_stream_t stream,
                                     const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || codes_out == nullptr || act_amax == nullptr)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && (cfg->tile_n != 0 || cfg->reserved != 0)) return B200Q_ERR_INVALID;
  if (M < 0 || N < 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 16 != 0 || N % 256 != 0) return B200Q_ERR_INVALID;
  if ((a_scales_numel != 1 && a_scales_numel != M) || (b_scales_numel != 1 && b_scales_numel != N)) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(codes_out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (M == 0 || N == 0) return B200Q_OK;
  gemm::Params p{};
  p.a_scales = a_scales;
  p.b_scales = b_scales;
  p.a_scale_stride = a_scales_numel == 1 ? 0 : 1;
  p.b_scale_stride = b_scales_numel == 1 ? 0 : 1;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = reinterpret_cast<__nv_bfloat16*>(codes_out);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K);
  p.silu_f = static_cast<int>(N / 2);
  p.act_amax = act_amax;
  p.act_scale_out = scale_out;
  p.status = gemm::device_status_word();
  if (p.status == nullptr) return B200Q_ERR_CUDA;
  return gemm::launch_pair<false, 2>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream));
}

static int fill_rs(gemm::Params& p, gemm::RsTargets& rs, const b200q_peers* peers, int64_t M) {
  if (peers == nullptr || peers->world < 2 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world) return B200Q_ERR_INVALID;
  if (M % (static_cast<int64_t>(peers->world) * 128) != 0) return B200Q_ERR_INVALID;
  p.rs_world = peers->world;
  p.rs_rank = peers->rank;
  p.rs_rows = static_cast<int>(M / peers->world);
  for (int r = 0; r < peers->world; ++r) {
    if (peers->recv[r] == nullptr) return B200Q_ERR_INVALID;
    if (!aligned(peers->recv[r], 16)) return B200Q_ERR_ALIGN;
    rs.recv[r] = peers->recv[r];
  }
  return B200Q_OK;
}

int b200q_fp8_gemm_reduce_scatter(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel, const uint8_t* b_codes,
                                  const float* b_scales, int64_t b_scales_numel, const b200q_peers* peers, int64_t M, int64_t N,
                                  int64_t K, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr) return B200Q_ERR_INVALID;
  if (cfg != nullptr && (!gemm::valid_tile_n(cfg->tile_n) || cfg->reserved != 0)) return B200Q_ERR_INVALID;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 16 != 0 || N % 8 != 0) return B200Q_ERR_INVALID;
  if ((a_scales_numel != 1 && a_scales_numel != M) || (b_scales_numel != 1 && b_scales_numel != N)) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16)) return B200Q_ERR_ALIGN;
  gemm::Params p{};
  gemm::RsTargets rs{};
  if (int rc = fill_rs(p, rs, peers, M)) return rc;
  if (int rc = check_arch()) return rc;
  p.a_scales = a_scales;
  p.b_scales = b_scales;
  p.a_scale_stride = a_scales_numel == 1 ? 0 : 1;
  p.b_scale_stride = b_scales_numel == 1 ? 0 : 1;
  p.out = static_cast<__nv_bfloat16*>(peers->recv[peers->rank]);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K);
  return gemm::launch<false>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream), cfg, &rs);
}

}  // extern "C"
