// Host side of the tcgen05 GEMMs: TMA tensor maps, tile-shape choice, launch.
#pragma once

#include <cuda.h>

#include "gemm_kernel_2cta.cuh"
#include "gemm_kernel_nvf4_pair.cuh"
#include "gemm_kernel_splitk.cuh"

namespace b200q {
namespace gemm {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled resolved through the runtime, so the library has no link-time
// dependency on libcuda.
EncodeTiledFn encode_tiled();

// Device status word shared by all GEMM launches of this process on the current device.
int* device_status_word();

// Row-major byte matrix [rows, row_bytes] -> tiles of box_rows x 128 bytes, 128-byte swizzle,
// out-of-bounds bytes read as zero.
inline int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return B200Q_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

// bf16 output [M, N] -> boxes of 32 rows x 64 columns (128 bytes), 128-byte swizzle.
inline int make_output_map(CUtensorMap* map, const void* base, int64_t M, int64_t N) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return B200Q_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(N) * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

// Receive buffers of the reduce-scatter epilogue: recv[r] is rank r's buffer
// [world][rows_per_rank][N] bf16, mapped into this process (peer memory).
struct RsTargets {
  void* recv[8];
};

// Output maps of a launch: the local output, or one map per destination rank.
inline int build_out_maps(OutMaps* maps, Params& p, const RsTargets* rs) {
  p.tma_store = (p.N % 8 == 0) ? 1 : 0;
  if (p.rs_world > 1) {
    if (rs == nullptr || !p.tma_store || p.rs_world > 8 || p.rs_rows % 128 != 0 || p.rs_rows * p.rs_world != p.M)
      return B200Q_ERR_INVALID;
    for (int r = 0; r < p.rs_world; ++r)
      if (int rc = make_output_map(&maps->m[r], rs->recv[r], static_cast<int64_t>(p.rs_world) * p.rs_rows, p.N)) return rc;
    return B200Q_OK;
  }
  if (p.tma_store) return make_output_map(&maps->m[0], p.out, p.M, p.N);
  return B200Q_OK;
}

template <bool NVF4, int BN>
int launch_tile(const uint8_t* a, const uint8_t* b, Params p, cudaStream_t st, const RsTargets* rs = nullptr) {
  using C = Cfg<NVF4, BN>;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(gemm_kernel<NVF4, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return B200Q_ERR_CUDA;
    configured[dev] = true;
  }
  CUtensorMap ta, tb;
  OutMaps tout = {};
  if (int rc = make_operand_map(&ta, a, p.M, p.k_bytes, kBM)) return rc;
  if (int rc = make_operand_map(&tb, b, p.N, p.k_bytes, BN)) return rc;
  if (int rc = build_out_maps(&tout, p, rs)) return rc;
  const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  const int threads = (NVF4 && p.sf_copier) ? kThreads + 32 : kThreads;   // optional scale-copier warp
  gemm_kernel<NVF4, BN><<<grid, threads, C::kSmemBytes, st>>>(ta, tb, tout, p);
  return check_launch();
}

// Swizzled block-scale buffer as a 3-D tensor [128 u32 = one 512-byte tile, column tile, row tile].
inline int make_scale_map(CUtensorMap* map, const void* base, int64_t row_tiles, int64_t col_tiles, int box_row_tiles) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return B200Q_ERR_CUDA;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(col_tiles), static_cast<cuuint64_t>(row_tiles)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(col_tiles) * 512};
  const cuuint32_t box[3] = {128, 4, static_cast<cuuint32_t>(box_row_tiles)};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

// CTA-pair kernel: clusters of two CTAs, one cluster per 256 x 256 output tile.
template <bool NVF4, int SILU = 0>
int launch_pair(const uint8_t* a, const uint8_t* b, Params p, cudaStream_t st, const RsTargets* rs = nullptr) {
  using C = Cfg2<NVF4>;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<NVF4, SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return B200Q_ERR_CUDA;
    configured[dev] = true;
  }
  CUtensorMap ta, tb, tsfa, tsfb;
  OutMaps tout = {};
  if (int rc = make_operand_map(&ta, a, p.M, p.k_bytes, 128)) return rc;
  if (int rc = make_operand_map(&tb, b, p.N, p.k_bytes, kPairN / 2)) return rc;
  if constexpr (SILU == 2) {
    // E4M3 codes [M, F] leave through plain stores: no output map
    p.tma_store = 0;
    if (rs != nullptr || p.rs_world > 1) return B200Q_ERR_INVALID;
  } else if constexpr (SILU == 1) {
    // out is [M, F]: TMA stores only (F is a multiple of 128)
    p.tma_store = 1;
    if (rs != nullptr || p.rs_world > 1) return B200Q_ERR_INVALID;
    if (int rc = make_output_map(&tout.m[0], p.out, p.M, p.silu_f)) return rc;
  } else {
    if (int rc = build_out_maps(&tout, p, rs)) return rc;
  }
  if constexpr (NVF4) {
    if (int rc = make_scale_map(&tsfa, p.sfa, (p.M + 127) / 128, p.sf_col_tiles, 1)) return rc;
    if (int rc = make_scale_map(&tsfb, p.sfb, (p.N + 127) / 128, p.sf_col_tiles, 2)) return rc;
  } else {
    tsfa = ta;
    tsfb = ta;
  }
  const int tiles = ((p.M + kPairM - 1) / kPairM) * (SILU ? (p.silu_f + kPairN / 2 - 1) / (kPairN / 2) : (p.N + kPairN - 1) / kPairN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pairs * 2));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_pair_kernel<NVF4, SILU>, ta, tb, tout, tsfa, tsfb, p) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return B200Q_OK;
}

// NVFP4 CTA-pair kernel with the scales stored to tensor memory by warps (gemm_kernel_nvf4_pair.cuh).
inline int launch_nvf4_pair(const uint8_t* a, const uint8_t* b, Params p, cudaStream_t st) {
  using C = CfgNvPair;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(gemm_nvf4_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return B200Q_ERR_CUDA;
    configured[dev] = true;
  }
  CUtensorMap ta, tb, tsfa, tsfb;
  if (int rc = make_operand_map(&ta, a, p.M, p.k_bytes, 128)) return rc;
  if (int rc = make_operand_map(&tb, b, p.N, p.k_bytes, 128)) return rc;
  if (int rc = make_scale_map(&tsfa, p.sfa, (p.M + 127) / 128, p.sf_col_tiles, 1)) return rc;
  if (int rc = make_scale_map(&tsfb, p.sfb, (p.N + 127) / 128, p.sf_col_tiles, 2)) return rc;
  const int tiles = ((p.M + kPairM - 1) / kPairM) * ((p.N + kPairN - 1) / kPairN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pairs * 2));
  cfg.blockDim = dim3(kNvPairThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_nvf4_pair_kernel<0>, ta, tb, tsfa, tsfb, p) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return B200Q_OK;
}

// Small-M kernel (M <= 128): operands swapped, one cluster of `splits` CTAs per tile of 128
// weight rows.  Up to one CTA per SM the operand ring takes all of shared memory; beyond that
// the ring is sized so that two CTAs share an SM, which lets one CTA's prologue and cluster
// reduction overlap the other's weight stream and fits twice as many CTAs into a wave.
// `stages` > 0 overrides the ring depth.
template <bool NVF4>
int launch_smallm(const uint8_t* a, const uint8_t* b, Params p, cudaStream_t st, int splits, int stages) {
  using C = SmallCfg<NVF4>;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(gemm_smallm_kernel<NVF4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
      return B200Q_ERR_CUDA;
    configured[dev] = true;
  }
  const int bt = ((p.M + 15) / 16) * 16;
  const int tiles = (p.N + kSmallWRows - 1) / kSmallWRows;
  const int most = C::max_stages(bt, kSmemLimit);
  if (stages <= 0) {
    stages = most;
    if (tiles * splits > sm_count()) {
      // two CTAs per SM: half of the SM's 228 KiB (1 KiB reserved per CTA) and, for NVFP4,
      // half of the 512 tensor-memory columns (128 accumulator + 32 scale columns per stage)
      stages = C::max_stages(bt, kSmallHalfSmem);
      if (NVF4 && stages > 4) stages = 4;
    }
  }
  if (stages > most) stages = most;
  if (stages < 2) stages = 2;
  CUtensorMap tw, tx;
  if (int rc = make_operand_map(&tw, b, p.N, p.k_bytes, kSmallWRows)) return rc;
  if (int rc = make_operand_map(&tx, a, p.M, p.k_bytes, bt)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * splits));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(C::smem_bytes(bt, stages));
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see common.cuh: pdl_wait in the kernel
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, gemm_smallm_kernel<NVF4>, tw, tx, p, splits, stages, bt) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return B200Q_OK;
}

// Cluster size of the small-M kernel.  Measured: one SM pulls about 60 bytes per nanosecond
// through TMA whatever the ring depth, so about 110 streaming SMs are needed to saturate HBM;
// the smallest power of two that reaches that many CTAs wins, larger clusters only add
// reduction cost.  With at most 32 tokens the partial tiles are small enough that two CTAs per SM
// pay (one's prologue and cluster reduction under the other's weight stream: 10-25 % faster at
// 16 tokens, neutral at 64, slower at 128), so the target there is one and a half CTAs per SM.
inline int smallm_splits(int n_tiles, int k_tiles, int sms, int tokens) {
  const int want = tokens <= 32 ? (sms * 3) / 2 : (sms * 3) / 4;
  int s = 1;
  while (s < 8 && n_tiles * s < want && s * 2 <= k_tiles) s <<= 1;
  return s;
}

bool valid_tile_n(int bn);    // values b200q_cfg::tile_n accepts
int sf_copier_enabled();     // environment variable B200Q_SF_COPIER (default in gemm_fp8.cu)
int forced_smallm_stages();  // from the environment variable B200Q_SMALLM_STAGES (0 when unset)

// Tile width: 256 when that still gives every SM a tile, else 128.  `cfg->tile_n` (128 / 256)
// overrides the choice (used by tests to cover both instantiations); 512 forces the CTA-pair
// kernel (256 x 256 tiles), which is otherwise used when there are at least sm_count/2 such tiles.
// M <= 128 goes to the small-M kernel unless a tile width is forced.
template <bool NVF4>
int launch(const uint8_t* a, const uint8_t* b, Params p, cudaStream_t st, const b200q_cfg* cfg, const RsTargets* rs = nullptr) {
  p.status = device_status_word();
  if (p.status == nullptr) return B200Q_ERR_CUDA;
  p.sf_copier = NVF4 ? sf_copier_enabled() : 0;
  p.static_weights = (cfg != nullptr && cfg->static_weights != 0) ? 1 : 0;
  int bn = cfg != nullptr ? cfg->tile_n : 0;
  const int k_tiles = (p.k_bytes + kBKBytes - 1) / kBKBytes;
  if (rs == nullptr && p.M <= kBM) {
    // small M: weights are streamed once; the swapped-operand cluster kernel handles it
    // (1001 / 1002 / 1004 / 1008 force 1 / 2 / 4 / 8 CTAs per tile)
    int splits = 0;
    if (bn == 1001 || bn == 1002 || bn == 1004 || bn == 1008) splits = bn - 1000;
    else if (bn == 0) splits = smallm_splits((p.N + kSmallWRows - 1) / kSmallWRows, k_tiles, sm_count(), p.M);
    if (splits >= 1 && splits <= k_tiles) return launch_smallm<NVF4>(a, b, p, st, splits, forced_smallm_stages());
  }
  if (bn >= 1000) bn = 0;
  const int64_t pair_tiles = static_cast<int64_t>((p.M + kPairM - 1) / kPairM) * ((p.N + kPairN - 1) / kPairN);
  // CTA-pair kernels (256 x 256 tiles) whenever they fill the SM pairs: measured 2.9 vs 2.75 PFLOP/s
  // for FP8 and 4.8 vs 3.4 for NVFP4 at 8192^3 against the single-CTA 128 x 256 tile.  The NVFP4 pair
  // kernel with the scale warps writes local output only; the reduce-scatter epilogue keeps the
  // generic kernels.
  if (bn == 512 || (bn == 0 && pair_tiles >= sm_count() / 2)) {
    if constexpr (NVF4) {
      if (rs == nullptr) return launch_nvf4_pair(a, b, p, st);
      if (bn == 512) return launch_pair<NVF4>(a, b, p, st, rs);
    } else {
      return launch_pair<NVF4>(a, b, p, st, rs);
    }
  }
  if (bn != 128 && bn != 256) {
    const int64_t tiles256 = static_cast<int64_t>((p.M + kBM - 1) / kBM) * ((p.N + 255) / 256);
    bn = (tiles256 >= sm_count()) ? 256 : 128;
  }
  return bn == 256 ? launch_tile<NVF4, 256>(a, b, p, st, rs) : launch_tile<NVF4, 128>(a, b, p, st, rs);
}

}  // namespace gemm
}  // namespace b200q
