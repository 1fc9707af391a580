// NVFP4 x NVFP4 block-scaled GEMM entry point (tcgen05 kind::mxf4nvf4.block_scale, block 16,
// UE4M3 scales read from the 128x4 swizzled layout the quantize kernel writes).
#include "gemm_host.cuh"

using namespace b200q;

extern "C" {

int b200q_nvfp4_gemm(const uint8_t* a_codes, const uint8_t* a_scales, const float* a_global, const uint8_t* b_codes,
                     const uint8_t* b_scales, const float* b_global, const void* bias, void* out, int64_t M, int64_t N,
                     int64_t K, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || a_global == nullptr ||
      b_global == nullptr || out == nullptr)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && (!gemm::valid_tile_n(cfg->tile_n) || cfg->reserved != 0)) return B200Q_ERR_INVALID;
  if (M < 0 || N < 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 32 != 0) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(a_scales, 16) || !aligned(b_scales, 16) || !aligned(out, 16))
    return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (M == 0 || N == 0) return B200Q_OK;
  gemm::Params p{};
  p.a_scales = a_global;
  p.b_scales = b_global;
  p.sfa = a_scales;
  p.sfb = b_scales;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K / 2);
  p.sf_col_tiles = static_cast<int>((K / 16 + 3) / 4);
  return gemm::launch<true>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream), cfg);
}

int b200q_nvfp4_gemm_reduce_scatter(const uint8_t* a_codes, const uint8_t* a_scales, const float* a_global, const uint8_t* b_codes,
                                    const uint8_t* b_scales, const float* b_global, const b200q_peers* peers, int64_t M, int64_t N,
                                    int64_t K, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || a_global == nullptr || b_global == nullptr)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && (!gemm::valid_tile_n(cfg->tile_n) || cfg->reserved != 0)) return B200Q_ERR_INVALID;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (K % 32 != 0 || N % 8 != 0) return B200Q_ERR_INVALID;
  if (peers == nullptr || peers->world < 2 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world) return B200Q_ERR_INVALID;
  if (M % (static_cast<int64_t>(peers->world) * 128) != 0) return B200Q_ERR_INVALID;
  if (!aligned(a_codes, 16) || !aligned(b_codes, 16) || !aligned(a_scales, 16) || !aligned(b_scales, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  gemm::Params p{};
  gemm::RsTargets rs{};
  p.rs_world = peers->world;
  p.rs_rank = peers->rank;
  p.rs_rows = static_cast<int>(M / peers->world);
  for (int r = 0; r < peers->world; ++r) {
    if (peers->recv[r] == nullptr) return B200Q_ERR_INVALID;
    if (!aligned(peers->recv[r], 16)) return B200Q_ERR_ALIGN;
    rs.recv[r] = peers->recv[r];
  }
  p.a_scales = a_global;
  p.b_scales = b_global;
  p.sfa = a_scales;
  p.sfb = b_scales;
  p.out = static_cast<__nv_bfloat16*>(peers->recv[peers->rank]);
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.k_bytes = static_cast<int>(K / 2);
  p.sf_col_tiles = static_cast<int>((K / 16 + 3) / 4);
  return gemm::launch<true>(a_codes, b_codes, p, static_cast<cudaStream_t>(stream), cfg, &rs);
}

}  // extern "C"
