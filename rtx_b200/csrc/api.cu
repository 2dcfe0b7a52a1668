// extern "C" entry points of librtxb: argument checks, tensor-map encoding and
// kernel launches.  No allocation, no synchronisation; everything is enqueued
// on the caller's stream.
#include "../../include/rtxb.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "gemm_blockscaled.cuh"
#include "gemm_skinny.cuh"

#include <atomic>
#include "quant.cuh"
#include "gemm_decode_fused.cuh"
#include "gemm_fused_quant.cuh"
#include "reduce.cuh"
#include "peer.cuh"

using namespace rtxb;

namespace {

thread_local char g_last_error[256] = "";

int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where, cudaGetErrorString(e));
  return RTXB_E_CUDA;
}
int fail_msg(int code, const char* msg) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", msg);
  return code;
}

#define RTXB_CHECK_LAUNCH(where)                                \
  do {                                                          \
    cudaError_t e__ = cudaGetLastError();                       \
    if (e__ != cudaSuccess) return fail_cuda(e__, where);       \
  } while (0)

}  // namespace

namespace rtxb {
// Records `msg` as this thread's error detail (what rtxb_last_cuda_error() returns) and hands `code`
// back; for the library's other translation units.
int set_last_error(int code, const char* msg) { return fail_msg(code, msg); }
}  // namespace rtxb

namespace {

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---- driver entry point for tensor-map encoding (no link-time libcuda) ----
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// ---- tensor maps --------------------------------------------------------------------------------
// A tensor map is a pure function of the base address, extents, strides and box, so encoded maps are
// kept in a small per-thread table and re-used by later launches on the same buffers (a decode step
// launches in microseconds; two to four driver encodes per launch were a visible part of that).
struct MapKey {
  const void* base;
  uint64_t dim[3];
  uint64_t stride[2];   // bytes, dimensions 1 and 2
  uint32_t box[3];
  uint32_t rank;        // 2 or 3
  uint32_t words;       // 0: bytes with the 128-byte swizzle (payload); 1: 32-bit words, no swizzle (scale tiles);
                        // 2 / 3: 16-bit / 32-bit elements with the 64-byte swizzle (output tiles of the epilogue)
};

struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool valid;
};

constexpr int kMapSlots = 64;
thread_local MapSlot t_map_cache[kMapSlots];

int encode_map(CUtensorMap* out, const MapKey& key, const char* what) {
  uint64_t h = reinterpret_cast<uintptr_t>(key.base) >> 4;
  h = h * 0x9E3779B97F4A7C15ull + key.dim[1] * 31 + key.dim[2] * 7 + key.box[1] * 131 + key.box[2] * 17 + key.rank +
      key.words * 3 + key.stride[1];
  MapSlot& slot = t_map_cache[(h >> 17) % kMapSlots];
  if (slot.valid && memcmp(&slot.key, &key, sizeof(MapKey)) == 0) {
    *out = slot.map;
    return RTXB_OK;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail_msg(RTXB_E_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t gdim[3] = {key.dim[0], key.dim[1], key.dim[2]};
  cuuint64_t gstride[2] = {key.stride[0], key.stride[1]};
  cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  static const CUtensorMapDataType kTypes[5] = {CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_DATA_TYPE_UINT32,
                                               CU_TENSOR_MAP_DATA_TYPE_UINT16, CU_TENSOR_MAP_DATA_TYPE_UINT32,
                                               CU_TENSOR_MAP_DATA_TYPE_UINT32};
  static const CUtensorMapSwizzle kSwizzles[5] = {CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_64B,
                                                  CU_TENSOR_MAP_SWIZZLE_128B};
  const int kind = key.words < 5 ? key.words : 0;
  CUresult r = fn(out, kTypes[kind], key.rank, const_cast<void*>(key.base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, kSwizzles[kind], CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what,
             static_cast<int>(r));
    return RTXB_E_DRIVER;
  }
  slot.key = key;
  slot.map = *out;
  slot.valid = true;
  return RTXB_OK;
}

MapKey blank_key(const void* base) {
  MapKey k;
  memset(&k, 0, sizeof(k));   // padding bytes too: keys are compared with memcmp
  k.base = base;
  return k;
}

// byte matrix [rows, row_bytes] (pitch row_bytes), boxes of 128 bytes x box_rows, 128-byte swizzle,
// out-of-range elements read as zero
int make_payload_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  if (!aligned(base, 16) || row_bytes % 16 != 0) return fail_msg(RTXB_E_ALIGNMENT, "payload must be 16-byte aligned");
  MapKey k = blank_key(base);
  k.rank = 2;
  k.dim[0] = static_cast<uint64_t>(row_bytes);
  k.dim[1] = static_cast<uint64_t>(rows);
  k.stride[0] = static_cast<uint64_t>(row_bytes);
  k.box[0] = 128u;
  k.box[1] = static_cast<uint32_t>(box_rows);
  return encode_map(map, k, "payload");
}

// the same byte matrix viewed as [row_bytes / 128][rows][128]: boxes of `box_k` consecutive 128-byte
// K chunks x box_rows rows, each chunk landing as its own swizzled tile.  Needs row_bytes % 128 == 0
// (otherwise the last chunk of a row would run into the next row instead of reading zeros).
int make_payload_map_ksteps(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int box_rows,
                            int box_k) {
  if (!aligned(base, 16) || row_bytes % 128 != 0) return fail_msg(RTXB_E_ALIGNMENT, "payload rows must be 128-byte multiples");
  MapKey k = blank_key(base);
  k.rank = 3;
  k.dim[0] = 128u;
  k.dim[1] = static_cast<uint64_t>(rows);
  k.dim[2] = static_cast<uint64_t>(row_bytes / 128);
  k.stride[0] = static_cast<uint64_t>(row_bytes);
  k.stride[1] = 128u;
  k.box[0] = 128u;
  k.box[1] = static_cast<uint32_t>(box_rows);
  k.box[2] = static_cast<uint32_t>(box_k);
  return encode_map(map, k, "payload K steps");
}

// scale tiles as a matrix of 512-byte rows (128 x uint32), boxes of `box_rows` consecutive tiles
int make_scale_map(CUtensorMap* map, const void* base, int64_t total_tiles, int box_rows) {
  MapKey k = blank_key(base);
  k.rank = 2;
  k.words = 1;
  k.dim[0] = 128u;
  k.dim[1] = static_cast<uint64_t>(total_tiles);
  k.stride[0] = 512u;
  k.box[0] = 128u;
  k.box[1] = static_cast<uint32_t>(box_rows);
  return encode_map(map, k, "scales");
}

// scale tiles of B for the pair kernel: [2 halves][rows = 512-byte tiles][128 words], the second half
// `delta_tiles` tiles after the first, so one box brings the tiles of both 128-row blocks behind a
// 256-wide accumulator tile.  Rows are limited to those whose second half lies inside the buffer.
int make_scale_map_halves(CUtensorMap* map, const void* base, int64_t total_tiles, int box_rows, int64_t delta_tiles) {
  MapKey k = blank_key(base);
  k.rank = 3;
  k.words = 1;
  k.dim[0] = 128u;
  k.dim[1] = static_cast<uint64_t>(total_tiles - delta_tiles);
  k.dim[2] = 2u;
  k.stride[0] = 512u;
  k.stride[1] = static_cast<uint64_t>(delta_tiles) * 512u;
  k.box[0] = 128u;
  k.box[1] = static_cast<uint32_t>(box_rows);
  k.box[2] = 2u;
  return encode_map(map, k, "scale halves");
}

// output matrix [rows, cols] of 2- or 4-byte elements, row pitch ldo elements; one box = the 32 rows x 32 columns an
// epilogue warp stages per store: 64-byte rows with the 64-byte swizzle (BF16), 128-byte rows with the 128-byte
// swizzle (FP32: whole 128-byte lines, also over NVLink); stores are clipped at the edges
int make_out_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ldo, int elem_bytes) {
  MapKey k = blank_key(base);
  k.rank = 2;
  k.words = elem_bytes == 2 ? 2 : 4;
  k.dim[0] = static_cast<uint64_t>(cols);
  k.dim[1] = static_cast<uint64_t>(rows);
  k.stride[0] = static_cast<uint64_t>(ldo) * elem_bytes;
  k.box[0] = 32u;
  k.box[1] = 32u;
  return encode_map(map, k, "output");
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device instead of per launch
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Done { const void* kernel; int device; int bytes; };
  static std::mutex mu;
  static std::vector<Done> done;
  thread_local Done last = {nullptr, -1, 0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (last.kernel == kernel && last.device == dev && last.bytes >= bytes) return cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Done& d : done)
      if (d.kernel == kernel && d.device == dev && d.bytes >= bytes) {
        last = d;
        return cudaSuccess;
      }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done.push_back({kernel, dev, bytes});
    last = done.back();
  }
  return cudaSuccess;
}

// SMs the persistent kernels leave free (for a collective that runs beside them); process-wide
std::atomic<int> g_sm_margin{0};

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  int n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    if (cached[dev] == 0) {
      int q = 0;
      if (cudaDeviceGetAttribute(&q, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || q <= 0) q = 148;
      cached[dev] = q;
    }
    n = cached[dev];
  }
  const int usable = n - g_sm_margin.load(std::memory_order_relaxed);
  return usable < 2 ? 2 : usable;
}

// launch `kernel` so that it may start while the kernel before it on the stream is still running
// (both sides use griddepcontrol to order their memory accesses)
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                             bool dependent, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Caller-selected GEMM schedule of this thread (0 = the library chooses): 1 single-CTA 128 x 256 tiles,
// 2 CTA pairs with 256 x 256 tiles, 3 streaming 128 x 64 tiles (only for M <= 128, else ignored),
// 4 CTA pairs that quantize the activation operand themselves (composite MXFP8 forwards only; the
// packed-operand GEMM entry points treat it as 2).
thread_local int t_gemm_schedule = 0;

// Schedule choice: the CTA-pair kernel (256 x 256 pair tiles) unless the problem has a single
// 128-row block of A, where half of every pair would idle.
bool use_pair_kernel(int m_tiles) {
  if (t_gemm_schedule == 1 || t_gemm_schedule == 3) return false;
  if (t_gemm_schedule == 2 || t_gemm_schedule == 4) return true;
  return m_tiles >= 2;
}

// M <= 128 and too few 256-wide tiles to occupy the SMs: the 128 x 64 skinny kernel.  With many
// 256-wide tiles (N >= ~19k) the large-tile kernel already keeps more bytes in flight per SM and
// streams faster.
bool use_skinny_kernel(int m_tiles, int64_t n_rows_b) {
  if (m_tiles != 1) return false;
  if (t_gemm_schedule == 3) return true;
  if (t_gemm_schedule == 1 || t_gemm_schedule == 2 || t_gemm_schedule == 4) return false;
  return (n_rows_b + kBlockN - 1) / kBlockN < 74;
}

// output split into blocks of rows, each block its own buffer (pair kernel, TMA-store epilogue)
struct BlockOutputs {
  void* const* bases;   // n_blocks buffers of [block_rows, out_cols] elements, pitch ldo
  int n_blocks;
  int64_t block_rows;   // multiple of 256
  int first_block;      // the tile order starts at the raster group that holds this block
};

// outer scales of the NVFP4 row-region policy (kEpiRegionBf16)
struct RegionScales {
  const float* x;
  const float* w;
  int x_rows, w_rows;
};

template <int KIND, int EPI>
int launch_gemm(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n_rows_b,
                int64_t row_bytes, int64_t sf_k_chunks, int64_t ldo, int64_t out_cols, int64_t glu_inter,
                const float* out_scale, cudaStream_t stream, int* status, void* q_out = nullptr,
                void* sf_out = nullptr, bool overlap_previous = false, const RegionScales* regions = nullptr,
                const BlockOutputs* blocks = nullptr, bool after_quantizer = false) {
  // after_quantizer: EVERY operand comes from the kernel enqueued just before this one (the composite forwards'
  // quantizer); the pair and single-CTA kernels are then launched as programmatic dependents — they wait for that
  // grid before their first load, their set-up runs beside its tail.  The streaming kernel is launched normally.
  // overlap_previous: B and its scales do not depend on the kernel launched just before this one on
  // the stream, so the streaming kernel may start fetching them while that kernel is still running
  using T = GemmTraits<KIND>;
  CUtensorMap map_a, map_b;
  int rc = make_payload_map(&map_a, qa, m, row_bytes, 128);
  if (rc) return rc;
  rc = make_payload_map(&map_b, qb, n_rows_b, row_bytes, 128);
  if (rc) return rc;
  GemmParams p;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n_rows_b);
  p.k_tiles = static_cast<int>((row_bytes + kBlockKBytes - 1) / kBlockKBytes);
  p.m_tiles = static_cast<int>((m + kBlockM - 1) / kBlockM);
  p.n_tiles = glu_inter ? static_cast<int>((glu_inter + 127) / 128) : static_cast<int>((n_rows_b + kBlockN - 1) / kBlockN);
  p.glu_inter = static_cast<int>(glu_inter);
  p.group_m = p.m_tiles;  // refined per kernel below
  p.sfa = static_cast<const uint8_t*>(sa);
  p.sfb = static_cast<const uint8_t*>(sb);
  p.sf_k_chunks = static_cast<int>(sf_k_chunks);
  p.out = out;
  p.ldo = ldo;
  p.out_cols = static_cast<int>(out_cols);
  p.out_vec_ok = (aligned(out, 16) && (ldo * (EPI == kEpiF32 ? 4 : 2)) % 16 == 0) ? 1 : 0;
  p.tma_out = 0;
  p.out_block_rows = 0;
  p.tile_shift = 0;
  p.out_scale = out_scale;
  p.x_region_scales = regions ? regions->x : nullptr;
  p.w_region_scales = regions ? regions->w : nullptr;
  p.x_region_rows = regions ? regions->x_rows : 1;
  p.w_region_rows = regions ? regions->w_rows : 1;
  p.q_out = static_cast<uint8_t*>(q_out);
  p.sf_out = static_cast<uint8_t*>(sf_out);
  p.sf_out_chunks = static_cast<int>((out_cols / 32 + 3) / 4);
  p.status = status;
  p.a_box_rows = 128;
  p.slots = 0;
  p.ks = 1;
  p.map3d = 0;
  p.sfb3d = 0;
  p.b_box256 = 0;
  p.overlap_previous = overlap_previous ? 1 : 0;
  if (blocks != nullptr && !use_pair_kernel(p.m_tiles))
    return fail_msg(RTXB_E_UNSUPPORTED, "block outputs are served by the CTA-pair kernel only");
  if (blocks == nullptr && use_skinny_kernel(p.m_tiles, n_rows_b) && !epi_is_glu(EPI) && EPI != kEpiRegionBf16) {
    // one 128-row block of A: the bandwidth-shaped 128 x 64 kernel streams B once over all SMs
    using S = SkinnyTraits<KIND>;
    p.a_box_rows = static_cast<int>(round_up(m, 8));
    // K steps per ring slot: as many as still leave four slots (one TMA instruction per operand and slot)
    p.map3d = row_bytes % 128 == 0 ? 1 : 0;
    p.ks = 1;
    if (p.map3d) {
      for (int ks = 4; ks >= 2; ks >>= 1)
        if (S::slots_for(p.a_box_rows, ks) >= 4 && p.k_tiles >= ks) { p.ks = ks; break; }
    }
    p.slots = S::slots_for(p.a_box_rows, p.ks);
    if (p.map3d) {
      rc = make_payload_map_ksteps(&map_a, qa, m, row_bytes, p.a_box_rows, p.ks);
      if (rc) return rc;
      rc = make_payload_map_ksteps(&map_b, qb, n_rows_b, row_bytes, kSkinnyN, p.ks);
      if (rc) return rc;
    } else {
      rc = make_payload_map(&map_a, qa, m, row_bytes, p.a_box_rows);
      if (rc) return rc;
      rc = make_payload_map(&map_b, qb, n_rows_b, row_bytes, kSkinnyN);
      if (rc) return rc;
    }
    p.n_tiles = static_cast<int>((n_rows_b + kSkinnyN - 1) / kSkinnyN);
    auto sk = gemm_skinny_kernel<KIND, EPI == kEpiF32 ? kEpiF32 : kEpiBf16>;
    cudaError_t se = ensure_dynamic_smem(reinterpret_cast<const void*>(sk), kSkinnySmemBudget);
    if (se != cudaSuccess) return fail_cuda(se, "cudaFuncSetAttribute(skinny gemm)");
    se = launch_dependent(sk, p.n_tiles < sm_count() ? p.n_tiles : sm_count(), kGemmThreads,
                          S::smem_bytes(p.a_box_rows, p.ks, p.slots), stream, overlap_previous, map_a, map_b, p);
    if (se != cudaSuccess) return fail_cuda(se, "gemm_skinny_kernel launch");
    return RTXB_OK;
  }
  if (use_pair_kernel(p.m_tiles)) {
    using P = PairTraits<KIND>;
    constexpr int KS = P::kStepsPerBarrierP;
    CUtensorMap map_sfa, map_sfb;
    // BF16 / FP32 tiles leave through shared memory and TMA stores when the output can be described by a
    // tensor map (16-byte aligned base and pitch); ragged pitches keep the direct stores
    OutMaps maps_out = {};
    p.tma_out = (!epi_is_glu(EPI) && out != nullptr && p.out_vec_ok) ? 1 : 0;
    if (blocks != nullptr) {
      if (!p.tma_out) return fail_msg(RTXB_E_ALIGNMENT, "block outputs need 16-byte aligned buffers and pitch");
      for (int b = 0; b < blocks->n_blocks; ++b) {
        const int64_t rows_b = m - b * blocks->block_rows < blocks->block_rows ? m - b * blocks->block_rows : blocks->block_rows;
        if (!aligned(blocks->bases[b], 16)) return fail_msg(RTXB_E_ALIGNMENT, "block outputs must be 16-byte aligned");
        rc = make_out_map(&maps_out.m[b], blocks->bases[b], rows_b, out_cols, ldo, EPI == kEpiF32 ? 4 : 2);
        if (rc) return rc;
      }
      p.out_block_rows = static_cast<int>(blocks->block_rows);
    } else if (p.tma_out) {
      rc = make_out_map(&maps_out.m[0], out, m, out_cols, ldo, EPI == kEpiF32 ? 4 : 2);
      if (rc) return rc;
    }
    // one load per operand brings the KS K steps of a barrier group
    p.map3d = row_bytes % 128 == 0 ? 1 : 0;
    if (p.map3d) {
      rc = make_payload_map_ksteps(&map_a, qa, m, row_bytes, 128, KS);
      if (rc) return rc;
      rc = make_payload_map_ksteps(&map_b, qb, n_rows_b, row_bytes, 128, KS);
      if (rc) return rc;
    }
    rc = make_scale_map(&map_sfa, sa, static_cast<int64_t>(p.m_tiles) * sf_k_chunks, KS * P::kSfChunks);
    if (rc) return rc;
    // both halves of a 256-wide tile in one box when the second half always exists
    const int64_t b_blocks = (n_rows_b + 127) / 128;
    const int64_t half_delta = glu_inter ? glu_inter / 128 : 1;
    p.sfb3d = (glu_inter ? (glu_inter % 128 == 0 && n_rows_b == 2 * glu_inter) : (b_blocks % 2 == 0)) ? 1 : 0;
    if (p.sfb3d)
      rc = make_scale_map_halves(&map_sfb, sb, b_blocks * sf_k_chunks, KS * P::kSfChunks, half_delta * sf_k_chunks);
    else
      rc = make_scale_map(&map_sfb, sb, b_blocks * sf_k_chunks, KS * P::kSfChunks);
    if (rc) return rc;
    auto pk = gemm_blockscaled_pair_kernel<KIND, EPI>;
    cudaError_t pe = ensure_dynamic_smem(reinterpret_cast<const void*>(pk), P::kSmemBytes);
    if (pe != cudaSuccess) return fail_cuda(pe, "cudaFuncSetAttribute(pair gemm)");
    {
      // A panel of a raster group: about 32 MB (group_m pairs x 256 rows x row_bytes) so that it stays in L2
      const int m_pairs = (p.m_tiles + 1) / 2;
      int64_t g = (32ll << 20) / (256 * row_bytes);
      p.group_m = static_cast<int>(g < 4 ? 4 : (g > m_pairs ? m_pairs : g));
    }
    const int64_t pair_tiles = static_cast<int64_t>((p.m_tiles + 1) / 2) * p.n_tiles;
    const int max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(pair_tiles < max_pairs ? pair_tiles : max_pairs);
    if (blocks != nullptr) {
      const int64_t start_pair = static_cast<int64_t>(blocks->first_block) * (blocks->block_rows / 256);
      p.tile_shift = static_cast<int>(((start_pair / p.group_m) * p.group_m * p.n_tiles) % pair_tiles);
    }
    cudaError_t le = launch_dependent(pk, 2 * pairs, kGemmThreads, P::kSmemBytes, stream,
                                      overlap_previous || after_quantizer, map_a, map_b, map_sfa, map_sfb, maps_out, p);
    if (le != cudaSuccess) return fail_cuda(le, "gemm_blockscaled_pair_kernel launch");
    return RTXB_OK;
  }
  if (p.m_tiles == 1) {
    // one row block: fetch only the live rows of A
    p.a_box_rows = static_cast<int>(round_up(m, 8));
    rc = make_payload_map(&map_a, qa, m, row_bytes, p.a_box_rows);
    if (rc) return rc;
  }
  if (!epi_is_glu(EPI)) {
    // plain tiles: the two 128-row halves of B are consecutive rows, one 256-row box brings both
    p.b_box256 = 1;
    rc = make_payload_map(&map_b, qb, n_rows_b, row_bytes, 256);
    if (rc) return rc;
  }
  auto kernel = gemm_blockscaled_kernel<KIND, EPI>;
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), T::kSmemBytes);
  if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(gemm)");
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  e = launch_dependent(kernel, grid, kGemmThreads, T::kSmemBytes, stream, overlap_previous || after_quantizer, map_a, map_b,
                       p);
  if (e != cudaSuccess) return fail_cuda(e, "gemm_blockscaled_kernel launch");
  return RTXB_OK;
}

// The one-kernel decode forward: up to four rows (every CTA re-quantizes all of X, which costs about
// 0.9 us per row even with twelve quantizer warps: measured 12.7 us at M = 1 and 18.7 us at M = 8 against
// 16.1 us for the three chained launches), K a multiple of 256 values whose quantized form (A tiles +
// scale tiles for every K step) leaves room for at least three ring slots of weights, and few enough
// 256-wide column tiles that the 64-wide streaming tiling is the right one.
bool decode_fused_eligible(const void* x, int64_t m, int64_t n, int64_t k) {
  if (t_gemm_schedule == 1 || t_gemm_schedule == 2 || t_gemm_schedule == 4) return false;
  if (m > 4 || k % 256 != 0 || !aligned(x, 16)) return false;
  const int k_tiles = static_cast<int>(k / 256);
  if (k_tiles < 2 || fused_slots_for(k_tiles, 2) < 3) return false;
  return use_skinny_kernel(1, n);
}

int launch_decode_fused(const void* x, const void* qw, const void* sw, const float* w_scale, void* out, int64_t m,
                        int64_t n, int64_t k, int scale_mode, float* x_scale_out, cudaStream_t stream, int* status) {
  using S = SkinnyTraits<kKindNvfp4>;
  const int64_t row_bytes = k / 2;
  GemmParams p = {};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k_tiles = static_cast<int>(k / 256);
  p.m_tiles = 1;
  p.n_tiles = static_cast<int>((n + kSkinnyN - 1) / kSkinnyN);
  p.sfb = static_cast<const uint8_t*>(sw);
  p.sf_k_chunks = static_cast<int>(round_up((k / 16 + 3) / 4, 4));
  p.out = out;
  p.ldo = n;
  p.out_cols = static_cast<int>(n);
  p.out_vec_ok = (aligned(out, 16) && (n * 2) % 16 == 0) ? 1 : 0;
  p.status = status;
  p.ks = fused_slots_for(p.k_tiles, 4) >= 4 && p.k_tiles >= 4 ? 4 : 2;
  p.slots = fused_slots_for(p.k_tiles, p.ks);
  p.map3d = 1;
  CUtensorMap map_b;
  int rc = make_payload_map_ksteps(&map_b, qw, n, row_bytes, kSkinnyN, p.ks);
  if (rc) return rc;
  FusedXParams fx;
  fx.x = static_cast<const __nv_bfloat16*>(x);
  fx.ldx = k;
  fx.k = static_cast<int>(k);
  fx.mode = scale_mode;
  fx.w_scale = w_scale;
  fx.x_scale_out = x_scale_out;
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_decode_fused_kernel), kSkinnySmemBudget);
  if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(decode fused)");
  // quantizer warps: 4 (they are also the epilogue warps) for one or two rows, 12 above
  const int threads = m <= 2 ? kGemmThreads : kFusedMaxThreads;
  e = launch_dependent(gemm_decode_fused_kernel, p.n_tiles < sm_count() ? p.n_tiles : sm_count(), threads,
                       fused_smem_bytes(p.k_tiles, p.ks, p.slots), stream, true, map_b, p, fx);
  if (e != cudaSuccess) return fail_cuda(e, "gemm_decode_fused_kernel launch");
  (void)S::kSfBytes;
  return RTXB_OK;
}

// The pair GEMM that quantizes A = X (BF16) in the kernel; B packed.  `row_bytes` = padded K.
template <int EPI>
int launch_fused_a(const void* x, int64_t ldx, const void* qb, const void* sb, void* out, int64_t m, int64_t n_rows_b,
                   int64_t k, int64_t ldo, int64_t out_cols, int64_t glu_inter, int rounding, cudaStream_t stream,
                   int* status, void* q_out = nullptr, void* sf_out = nullptr) {
  using P = PairTraits<kKindMxfp8>;
  constexpr int KS = P::kStepsPerBarrierP;
  const int64_t row_bytes = round_up(k, 32);
  const int64_t sf_k_chunks = (row_bytes / 32 + 3) / 4;
  GemmParams p = {};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n_rows_b);
  p.k_tiles = static_cast<int>((row_bytes + kBlockKBytes - 1) / kBlockKBytes);
  p.m_tiles = static_cast<int>((m + kBlockM - 1) / kBlockM);
  p.n_tiles = glu_inter ? static_cast<int>((glu_inter + 127) / 128) : static_cast<int>((n_rows_b + kBlockN - 1) / kBlockN);
  p.glu_inter = static_cast<int>(glu_inter);
  p.sfb = static_cast<const uint8_t*>(sb);
  p.sf_k_chunks = static_cast<int>(sf_k_chunks);
  p.out = out;
  p.ldo = ldo;
  p.out_cols = static_cast<int>(out_cols);
  p.out_vec_ok = (aligned(out, 16) && (ldo * 2) % 16 == 0) ? 1 : 0;
  p.x_region_rows = p.w_region_rows = 1;
  p.q_out = static_cast<uint8_t*>(q_out);
  p.sf_out = static_cast<uint8_t*>(sf_out);
  p.sf_out_chunks = static_cast<int>((out_cols / 32 + 3) / 4);
  p.status = status;
  p.a_box_rows = 128;
  p.ks = 1;
  CUtensorMap map_b, map_sfb;
  int rc;
  p.map3d = row_bytes % 128 == 0 ? 1 : 0;
  if (p.map3d) rc = make_payload_map_ksteps(&map_b, qb, n_rows_b, row_bytes, 128, KS);
  else rc = make_payload_map(&map_b, qb, n_rows_b, row_bytes, 128);
  if (rc) return rc;
  const int64_t b_blocks = (n_rows_b + 127) / 128;
  const int64_t half_delta = glu_inter ? glu_inter / 128 : 1;
  p.sfb3d = (glu_inter ? (glu_inter % 128 == 0 && n_rows_b == 2 * glu_inter) : (b_blocks % 2 == 0)) ? 1 : 0;
  if (p.sfb3d) rc = make_scale_map_halves(&map_sfb, sb, b_blocks * sf_k_chunks, KS * P::kSfChunks, half_delta * sf_k_chunks);
  else rc = make_scale_map(&map_sfb, sb, b_blocks * sf_k_chunks, KS * P::kSfChunks);
  if (rc) return rc;
  FusedAParams fa;
  fa.x = static_cast<const __nv_bfloat16*>(x);
  fa.ldx = ldx;
  fa.k = static_cast<int>(k);
  fa.vec_ok = (aligned(x, 16) && ldx % 8 == 0) ? 1 : 0;
  fa.round_to_infinity = rounding != RTXB_ROUND_FLOOR;
  auto kernel = gemm_mxfp8_fused_a_pair_kernel<EPI>;
  cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), P::kSmemBytes);
  if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(fused-A gemm)");
  const int m_pairs = (p.m_tiles + 1) / 2;
  int64_t g = (32ll << 20) / (256 * 2 * row_bytes);    // the A panel of a raster group is BF16 here
  p.group_m = static_cast<int>(g < 4 ? 4 : (g > m_pairs ? m_pairs : g));
  const int64_t pair_tiles = static_cast<int64_t>(m_pairs) * p.n_tiles;
  const int max_pairs = sm_count() / 2;
  const int pairs = static_cast<int>(pair_tiles < max_pairs ? pair_tiles : max_pairs);
  kernel<<<2 * pairs, kFusedQuantThreads, P::kSmemBytes, stream>>>(map_b, map_sfb, p, fa);
  RTXB_CHECK_LAUNCH("gemm_mxfp8_fused_a_pair_kernel");
  return RTXB_OK;
}

int check_gemm_args(const void* qa, const void* sa, const void* qb, const void* sb, const void* out, int64_t m,
                    int64_t n, int64_t k, int64_t ldo, int64_t out_cols, int out_elem_bytes) {
  if (!qa || !sa || !qb || !sb || !out) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || k <= 0) return fail_msg(RTXB_E_INVALID_ARGUMENT, "m, n, k must be positive");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (ldo < out_cols) return fail_msg(RTXB_E_INVALID_ARGUMENT, "output pitch smaller than its width");
  if (!aligned(sa, 16) || !aligned(sb, 16)) return fail_msg(RTXB_E_ALIGNMENT, "scale tiles must be 16-byte aligned");
  if (!aligned(out, out_elem_bytes)) return fail_msg(RTXB_E_ALIGNMENT, "output pointer is not element aligned");
  return RTXB_OK;
}

// grid-stride kernels: one wave of resident CTAs (per_sm = CTAs that fit one SM).  Fewer CTAs with equal tile
// counts (no straggler round) were measured slower: these kernels are bound by the loads in flight, and 8 %
// fewer CTAs cost 8 % of the rate (row quantizer 41.5 against 37.6 us on 16384 x 4096).
int quant_grid(int64_t tiles, int per_sm) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
  return static_cast<int>(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
}

struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<uint8_t*>(p)) {}
  uint8_t* take(size_t bytes) {
    uint8_t* r = base ? base + off : nullptr;
    off += static_cast<size_t>(round_up(static_cast<int64_t>(bytes), 256));
    return r;
  }
};

}  // namespace

extern "C" {

int rtxb_version(void) { return 100; }

int rtxb_set_sm_margin(int sms) {
  if (sms < 0 || sms > 128) return fail_msg(RTXB_E_INVALID_ARGUMENT, "SM margin must be in [0, 128]");
  g_sm_margin.store(sms, std::memory_order_relaxed);
  return RTXB_OK;
}
int rtxb_get_sm_margin(void) { return g_sm_margin.load(std::memory_order_relaxed); }

int rtxb_set_gemm_schedule(int schedule) {
  if (schedule < RTXB_SCHEDULE_AUTO || schedule > RTXB_SCHEDULE_FUSED_X)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown GEMM schedule");
  t_gemm_schedule = schedule;
  return RTXB_OK;
}
int rtxb_get_gemm_schedule(void) { return t_gemm_schedule; }

const char* rtxb_error_string(int code) {
  switch (code) {
    case RTXB_OK: return "ok";
    case RTXB_E_INVALID_ARGUMENT: return "invalid argument";
    case RTXB_E_UNSUPPORTED: return "unsupported configuration";
    case RTXB_E_ALIGNMENT: return "pointer or pitch not aligned";
    case RTXB_E_WORKSPACE: return "workspace too small";
    case RTXB_E_CUDA: return "CUDA runtime error";
    case RTXB_E_DRIVER: return "CUDA driver error";
    case RTXB_E_SCRATCH_CAPACITY: return "shape exceeds the built-in scratch array of the no-allocation entry point";
    default: return "unknown error";
  }
}

const char* rtxb_last_cuda_error(void) { return g_last_error; }

int64_t rtxb_mxfp8_storage_k(int64_t k) { return round_up(k, 32); }
int64_t rtxb_nvfp4_storage_k(int64_t k) { return round_up(k, 32); }

size_t rtxb_mxfp8_scale_bytes(int64_t rows, int64_t k, int layout) {
  const int64_t nb = round_up(k, 32) / 32;
  if (layout == RTXB_SCALE_ROW_MAJOR) return static_cast<size_t>(rows * nb);
  if (layout == RTXB_SCALE_MMA128) return static_cast<size_t>(round_up(rows, 128) / 128 * ((nb + 3) / 4) * 512);
  return 0;
}

size_t rtxb_nvfp4_scale_bytes(int64_t rows, int64_t k, int layout) {
  const int64_t nb = round_up(k, 32) / 16;
  if (layout == RTXB_SCALE_ROW_MAJOR) return static_cast<size_t>(rows * nb);
  // tiles along K padded to whole 256-value GEMM K tiles (4 tiles of 64 values)
  if (layout == RTXB_SCALE_MMA128) return static_cast<size_t>(round_up(rows, 128) / 128 * round_up((nb + 3) / 4, 4) * 512);
  return 0;
}

// `beside_previous`: launched as a programmatic dependent that never waits, so it may run beside the kernel before it
// on the stream (which must not touch its operands)
static int mxfp8_quantize_impl(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                               int scale_layout, int rounding, void* stream, bool beside_previous);

int rtxb_mxfp8_quantize(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales, int scale_layout,
                        int rounding, void* stream) {
  return mxfp8_quantize_impl(src, rows, k, ld, q, scales, scale_layout, rounding, stream, false);
}

static int mxfp8_quantize_impl(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                               int scale_layout, int rounding, void* stream, bool beside_previous) {
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!src || !q || !scales) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (rows > INT32_MAX || k > INT32_MAX - 256) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantMxParams p;
  p.src = static_cast<const __nv_bfloat16*>(src);
  p.q = static_cast<uint8_t*>(q);
  p.scales = static_cast<uint8_t*>(scales);
  p.rows = static_cast<int>(rows);
  p.k = static_cast<int>(k);
  p.kp = static_cast<int>(round_up(k, 32));
  p.ld = ld;
  p.nb = p.kp / 32;
  p.sf_chunks = (p.nb + 3) / 4;
  p.layout = scale_layout;
  p.round_to_infinity = rounding != RTXB_ROUND_FLOOR;
  const int64_t tiles = ((rows + 127) / 128) * ((p.kp + 127) / 128);
  cudaError_t le = launch_dependent(quant_mxfp8_rows_kernel, quant_grid(tiles, 6), kQuantThreads, 0,
                                    static_cast<cudaStream_t>(stream), beside_previous, p);
  if (le != cudaSuccess) return fail_cuda(le, "quant_mxfp8_rows_kernel launch");
  return RTXB_OK;
}

// X [m, k] and W [n, k] (contiguous BF16) to mma128-scaled MXFP8 in one launch
static int mxfp8_quantize_pair(const void* x, int64_t m, const void* w, int64_t n, int64_t k, void* qx, void* sx, void* qw,
                               void* sw, int rounding, void* stream) {
  if (!x || !w || !qx || !sx || !qw || !sw) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || k <= 0) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX - 256) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (!aligned(qx, 16) || !aligned(qw, 16) || !aligned(sx, 16) || !aligned(sw, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "packed outputs must be 16-byte aligned");
  QuantMxParams p[2];
  const void* src[2] = {x, w};
  void* q[2] = {qx, qw};
  void* sc[2] = {sx, sw};
  const int64_t rows[2] = {m, n};
  int64_t tiles = 0;
  for (int i = 0; i < 2; ++i) {
    p[i] = QuantMxParams{};
    p[i].src = static_cast<const __nv_bfloat16*>(src[i]);
    p[i].q = static_cast<uint8_t*>(q[i]);
    p[i].scales = static_cast<uint8_t*>(sc[i]);
    p[i].rows = static_cast<int>(rows[i]);
    p[i].k = static_cast<int>(k);
    p[i].kp = static_cast<int>(round_up(k, 32));
    p[i].ld = k;
    p[i].nb = p[i].kp / 32;
    p[i].sf_chunks = (p[i].nb + 3) / 4;
    p[i].layout = RTXB_SCALE_MMA128;
    p[i].round_to_infinity = rounding != RTXB_ROUND_FLOOR;
    tiles += ((rows[i] + 127) / 128) * ((p[i].kp + 127) / 128);
  }
  quant_mxfp8_rows2_kernel<<<quant_grid(tiles, 6), kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(p[0], p[1]);
  RTXB_CHECK_LAUNCH("quant_mxfp8_rows2_kernel");
  return RTXB_OK;
}

int rtxb_mxfp8_quantize_transposed(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                                   int scale_layout, int rounding, void* stream) {
  if (!src || !q || !scales) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < rows) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (rows > INT32_MAX || k > INT32_MAX - 256) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q, 16)) return fail_msg(RTXB_E_ALIGNMENT, "q must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantMxTParams p;
  p.src = static_cast<const __nv_bfloat16*>(src);
  p.q = static_cast<uint8_t*>(q);
  p.scales = static_cast<uint8_t*>(scales);
  p.rows = static_cast<int>(rows);
  p.k = static_cast<int>(k);
  p.kp = static_cast<int>(round_up(k, 32));
  p.ld = ld;
  p.nb = p.kp / 32;
  p.sf_chunks = (p.nb + 3) / 4;
  p.layout = scale_layout;
  p.round_to_infinity = rounding != RTXB_ROUND_FLOOR;
  p.q_rows = nullptr;
  p.s_rows = nullptr;
  p.np = p.nb_rows = p.chunks_rows = 0;
  const int64_t tiles = ((rows + 127) / 128) * ((p.kp + 127) / 128);
  cudaError_t ae = ensure_dynamic_smem(reinterpret_cast<const void*>(quant_mxfp8_transposed_kernel<false>), kQtSmemBytes);
  if (ae != cudaSuccess) return fail_cuda(ae, "cudaFuncSetAttribute(transposed quantizer)");
  quant_mxfp8_transposed_kernel<false><<<quant_grid(tiles, kQtOccupancy), kQuantThreads, kQtSmemBytes,
                                         static_cast<cudaStream_t>(stream)>>>(p);
  RTXB_CHECK_LAUNCH("quant_mxfp8_transposed_kernel");
  return RTXB_OK;
}

int rtxb_mxfp8_quantize_dual(const void* src, int64_t m, int64_t n, int64_t ld, void* q_rows, void* s_rows, void* q_t,
                             void* s_t, int scale_layout, int rounding, void* stream) {
  if (!src || !q_rows || !s_rows || !q_t || !s_t) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || ld < n) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (m > INT32_MAX - 256 || n > INT32_MAX - 256) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q_rows, 16) || !aligned(q_t, 16)) return fail_msg(RTXB_E_ALIGNMENT, "payloads must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && (!aligned(s_rows, 16) || !aligned(s_t, 16)))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantMxTParams p;
  p.src = static_cast<const __nv_bfloat16*>(src);
  p.q = static_cast<uint8_t*>(q_t);          // transposed: [n, mp], blocks along m
  p.scales = static_cast<uint8_t*>(s_t);
  p.rows = static_cast<int>(n);
  p.k = static_cast<int>(m);
  p.kp = static_cast<int>(round_up(m, 32));
  p.ld = ld;
  p.nb = p.kp / 32;
  p.sf_chunks = (p.nb + 3) / 4;
  p.layout = scale_layout;
  p.round_to_infinity = rounding != RTXB_ROUND_FLOOR;
  p.q_rows = static_cast<uint8_t*>(q_rows);  // rows: [m, np], blocks along n
  p.s_rows = static_cast<uint8_t*>(s_rows);
  p.np = static_cast<int>(round_up(n, 32));
  p.nb_rows = p.np / 32;
  p.chunks_rows = (p.nb_rows + 3) / 4;
  const int64_t tiles = ((n + 127) / 128) * ((p.kp + 127) / 128);
  cudaError_t ae = ensure_dynamic_smem(reinterpret_cast<const void*>(quant_mxfp8_transposed_kernel<true>), kQtSmemBytes);
  if (ae != cudaSuccess) return fail_cuda(ae, "cudaFuncSetAttribute(dual quantizer)");
  quant_mxfp8_transposed_kernel<true><<<quant_grid(tiles, kQtOccupancy), kQuantThreads, kQtSmemBytes,
                                        static_cast<cudaStream_t>(stream)>>>(p);
  RTXB_CHECK_LAUNCH("quant_mxfp8_transposed_kernel<dual>");
  return RTXB_OK;
}

// rtxb_mxfp8_gemm; `after_quantizer`: launched as a programmatic dependent of the quantizer enqueued just before it
// (the kernels wait for that grid before they touch an operand; their set-up runs beside its tail)
static int mxfp8_gemm_impl(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n,
                           int64_t k, int64_t ldo, int out_dtype, void* stream, int* status, bool after_quantizer) {
  if (out_dtype != RTXB_OUT_BF16 && out_dtype != RTXB_OUT_F32)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown output dtype");
  int rc = check_gemm_args(qa, sa, qb, sb, out, m, n, k, ldo, n, out_dtype == RTXB_OUT_BF16 ? 2 : 4);
  if (rc) return rc;
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = (kp / 32 + 3) / 4;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == RTXB_OUT_BF16)
    return launch_gemm<kKindMxfp8, kEpiBf16>(qa, sa, qb, sb, out, m, n, kp, chunks, ldo, n, 0, nullptr, s, status, nullptr,
                                             nullptr, false, nullptr, nullptr, after_quantizer);
  return launch_gemm<kKindMxfp8, kEpiF32>(qa, sa, qb, sb, out, m, n, kp, chunks, ldo, n, 0, nullptr, s, status, nullptr,
                                          nullptr, false, nullptr, nullptr, after_quantizer);
}

int rtxb_mxfp8_gemm(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n,
                    int64_t k, int64_t ldo, int out_dtype, void* stream, int* status) {
  return mxfp8_gemm_impl(qa, sa, qb, sb, out, m, n, k, ldo, out_dtype, stream, status, false);
}

int rtxb_mxfp8_gemm_row_blocks(const void* qa, const void* sa, const void* qb, const void* sb, void* const* out_blocks,
                               int n_blocks, int64_t block_rows, int64_t m, int64_t n, int64_t k, int64_t ldo,
                               int out_dtype, int first_block, void* stream, int* status) {
  if (out_dtype != RTXB_OUT_BF16 && out_dtype != RTXB_OUT_F32)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown output dtype");
  if (!out_blocks || n_blocks < 1 || n_blocks > kMaxOutBlocks)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "between 1 and 8 output blocks");
  if (block_rows <= 0 || block_rows % 256 != 0 || (n_blocks - 1) * block_rows >= m || n_blocks * block_rows < m)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "blocks must be whole 256-row tiles that cover the m rows exactly");
  if (m < 256) return fail_msg(RTXB_E_UNSUPPORTED, "block outputs need at least one 256-row tile");
  for (int b = 0; b < n_blocks; ++b)
    if (!out_blocks[b]) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null output block");
  int rc = check_gemm_args(qa, sa, qb, sb, out_blocks[0], m, n, k, ldo, n, out_dtype == RTXB_OUT_BF16 ? 2 : 4);
  if (rc) return rc;
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = (kp / 32 + 3) / 4;
  const BlockOutputs blocks{out_blocks, n_blocks, block_rows, first_block < 0 ? 0 : first_block % n_blocks};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == RTXB_OUT_BF16)
    return launch_gemm<kKindMxfp8, kEpiBf16>(qa, sa, qb, sb, out_blocks[0], m, n, kp, chunks, ldo, n, 0, nullptr, s, status,
                                             nullptr, nullptr, false, nullptr, &blocks);
  return launch_gemm<kKindMxfp8, kEpiF32>(qa, sa, qb, sb, out_blocks[0], m, n, kp, chunks, ldo, n, 0, nullptr, s, status,
                                          nullptr, nullptr, false, nullptr, &blocks);
}

int rtxb_mxfp8_gemm_glu(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m,
                        int64_t inter, int64_t k, int64_t ldo, void* stream, int* status) {
  int rc = check_gemm_args(qa, sa, qb, sb, out, m, 2 * inter, k, ldo, inter, 2);
  if (rc) return rc;
  if (inter % 128 != 0) return fail_msg(RTXB_E_UNSUPPORTED, "fused GLU epilogue needs inter % 128 == 0");
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = (kp / 32 + 3) / 4;
  return launch_gemm<kKindMxfp8, kEpiGluBf16>(qa, sa, qb, sb, out, m, 2 * inter, kp, chunks, ldo, inter, inter, nullptr,
                                              static_cast<cudaStream_t>(stream), status);
}

int rtxb_mxfp8_gemm_glu_mx(const void* qa, const void* sa, const void* qb, const void* sb, void* h_bf16, void* q_h,
                           void* s_h, int64_t m, int64_t inter, int64_t k, int64_t ldo, void* stream, int* status) {
  if (!q_h || !s_h) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null packed output");
  int rc = check_gemm_args(qa, sa, qb, sb, q_h, m, 2 * inter, k, h_bf16 ? ldo : inter, inter, 1);
  if (rc) return rc;
  if (inter % 128 != 0) return fail_msg(RTXB_E_UNSUPPORTED, "fused GLU epilogue needs inter % 128 == 0");
  if (!aligned(q_h, 16) || !aligned(s_h, 16)) return fail_msg(RTXB_E_ALIGNMENT, "packed outputs must be 16-byte aligned");
  if (h_bf16 && !aligned(h_bf16, 2)) return fail_msg(RTXB_E_ALIGNMENT, "output pointer is not element aligned");
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = (kp / 32 + 3) / 4;
  return launch_gemm<kKindMxfp8, kEpiGluMx>(qa, sa, qb, sb, h_bf16, m, 2 * inter, kp, chunks, h_bf16 ? ldo : inter, inter,
                                            inter, nullptr, static_cast<cudaStream_t>(stream), status, q_h, s_h);
}

int rtxb_mxfp8_linear_fwd_fused_x(const void* x, int64_t ldx, const void* qw, const void* sw, void* out, int64_t m,
                                  int64_t n, int64_t k, int64_t ldo, int rounding, void* stream, int* status) {
  if (!x || !qw || !sw || !out) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || k <= 0 || ldx < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX - 256) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (ldo < n) return fail_msg(RTXB_E_INVALID_ARGUMENT, "output pitch smaller than its width");
  if (!aligned(sw, 16)) return fail_msg(RTXB_E_ALIGNMENT, "scale tiles must be 16-byte aligned");
  if (!aligned(out, 2) || !aligned(x, 2)) return fail_msg(RTXB_E_ALIGNMENT, "pointer is not element aligned");
  return launch_fused_a<kEpiBf16>(x, ldx, qw, sw, out, m, n, k, ldo, n, 0, rounding, static_cast<cudaStream_t>(stream),
                                  status);
}

int rtxb_mxfp8_gemm_glu_mx_fused_x(const void* x, int64_t ldx, const void* qb, const void* sb, void* h_bf16, void* q_h,
                                   void* s_h, int64_t m, int64_t inter, int64_t k, int64_t ldo, void* stream,
                                   int* status) {
  if (!x || !qb || !sb || !q_h || !s_h) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || inter <= 0 || k <= 0 || ldx < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (m > INT32_MAX || 2 * inter > INT32_MAX || k > INT32_MAX - 256)
    return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (inter % 128 != 0) return fail_msg(RTXB_E_UNSUPPORTED, "fused GLU epilogue needs inter % 128 == 0");
  if (!aligned(sb, 16) || !aligned(q_h, 16) || !aligned(s_h, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "scale tiles and packed outputs must be 16-byte aligned");
  if (h_bf16 && (!aligned(h_bf16, 2) || ldo < inter)) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad BF16 output");
  return launch_fused_a<kEpiGluMx>(x, ldx, qb, sb, h_bf16, m, 2 * inter, k, h_bf16 ? ldo : inter, inter, inter,
                                   RTXB_ROUND_INFINITY, static_cast<cudaStream_t>(stream), status, q_h, s_h);
}

size_t rtxb_mxfp8_linear_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  Carver c(nullptr);
  const int64_t kp = round_up(k, 32);
  c.take(m * kp);
  c.take(rtxb_mxfp8_scale_bytes(m, k, RTXB_SCALE_MMA128));
  c.take(n * kp);
  c.take(rtxb_mxfp8_scale_bytes(n, k, RTXB_SCALE_MMA128));
  return c.off;
}

int rtxb_mxfp8_linear_fwd(const void* x, const void* w, void* out, int64_t m, int64_t n, int64_t k, int rounding,
                          void* workspace, size_t workspace_bytes, void* stream, int* status) {
  if (!workspace || workspace_bytes < rtxb_mxfp8_linear_workspace_bytes(m, n, k))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_mxfp8_linear_fwd");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  Carver c(workspace);
  const int64_t kp = round_up(k, 32);
  uint8_t* qx = c.take(m * kp);
  uint8_t* sx = c.take(rtxb_mxfp8_scale_bytes(m, k, RTXB_SCALE_MMA128));
  uint8_t* qw = c.take(n * kp);
  uint8_t* sw = c.take(rtxb_mxfp8_scale_bytes(n, k, RTXB_SCALE_MMA128));
  int rc;
  if (t_gemm_schedule == RTXB_SCHEDULE_FUSED_X) {   // X is quantized by the GEMM's own quantizer warps
    if ((rc = rtxb_mxfp8_quantize(w, n, k, k, qw, sw, RTXB_SCALE_MMA128, rounding, stream))) return rc;
    return rtxb_mxfp8_linear_fwd_fused_x(x, k, qw, sw, out, m, n, k, n, rounding, stream, status);
  }
  // Both operands in ONE quantizer launch (the reference's dual quantizer), the GEMM behind it as a programmatic
  // dependent: two launches per forward instead of three, and the GEMM's set-up runs beside the quantizer's tail.
  // On small layers the launches, not the work, are the time.
  if ((rc = mxfp8_quantize_pair(x, m, w, n, k, qx, sx, qw, sw, rounding, stream))) return rc;
  return mxfp8_gemm_impl(qx, sx, qw, sw, out, m, n, k, n, RTXB_OUT_BF16, stream, status, true);
}

size_t rtxb_mxfp8_glu_mlp_workspace_bytes(int64_t m, int64_t k, int64_t inter, int64_t n_out) {
  Carver c(nullptr);
  const int64_t kp = round_up(k, 32), ip = round_up(inter, 32);
  c.take(m * kp);
  c.take(rtxb_mxfp8_scale_bytes(m, k, RTXB_SCALE_MMA128));
  c.take(2 * inter * kp);
  c.take(rtxb_mxfp8_scale_bytes(2 * inter, k, RTXB_SCALE_MMA128));
  c.take(m * ip);
  c.take(rtxb_mxfp8_scale_bytes(m, inter, RTXB_SCALE_MMA128));
  c.take(n_out * ip);
  c.take(rtxb_mxfp8_scale_bytes(n_out, inter, RTXB_SCALE_MMA128));
  return c.off;
}

int rtxb_mxfp8_glu_mlp_fwd(const void* x, const void* w_gu, const void* w_down, void* h, void* y, int64_t m, int64_t k,
                           int64_t inter, int64_t n_out, void* workspace, size_t workspace_bytes, void* stream,
                           int* status) {
  if (!workspace || workspace_bytes < rtxb_mxfp8_glu_mlp_workspace_bytes(m, k, inter, n_out))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_mxfp8_glu_mlp_fwd");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  if (inter % 128 != 0) return fail_msg(RTXB_E_UNSUPPORTED, "fused GLU epilogue needs inter % 128 == 0");
  Carver c(workspace);
  const int64_t kp = round_up(k, 32), ip = round_up(inter, 32);
  uint8_t* qx = c.take(m * kp);
  uint8_t* sx = c.take(rtxb_mxfp8_scale_bytes(m, k, RTXB_SCALE_MMA128));
  uint8_t* qg = c.take(2 * inter * kp);
  uint8_t* sg = c.take(rtxb_mxfp8_scale_bytes(2 * inter, k, RTXB_SCALE_MMA128));
  uint8_t* qh = c.take(m * ip);
  uint8_t* sh = c.take(rtxb_mxfp8_scale_bytes(m, inter, RTXB_SCALE_MMA128));
  uint8_t* qd = c.take(n_out * ip);
  uint8_t* sd = c.take(rtxb_mxfp8_scale_bytes(n_out, inter, RTXB_SCALE_MMA128));
  int rc;
  const bool fused_x = t_gemm_schedule == RTXB_SCHEDULE_FUSED_X;
  if (!fused_x && (rc = rtxb_mxfp8_quantize(x, m, k, k, qx, sx, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
    return rc;
  if ((rc = rtxb_mxfp8_quantize(w_gu, 2 * inter, k, k, qg, sg, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream))) return rc;
  // The down weight's quantizer (HBM bound, 40 registers, 0.5 KB of shared memory: its CTAs fit beside a GEMM CTA)
  // is launched AFTER the gate/up GEMM as a programmatic dependent that never waits: the GEMM releases its
  // dependents at entry, so the quantizer runs beside it.  Nothing the GEMM touches is read or written by it, and
  // the down GEMM (an ordinary launch) waits for both.  Measured: 0.231 against 0.248 ms per step at 1024 rows
  // (an eight-GPU shard), 0.610 against 0.643 at 4096, no difference at 8192 rows (power bound there).
  const bool beside = !fused_x;
  if (!beside &&
      (rc = rtxb_mxfp8_quantize(w_down, n_out, inter, inter, qd, sd, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
    return rc;
  // gate/up GEMM whose epilogue applies SiLU*up and writes H already quantized for the down projection
  // (and in BF16 too when the caller wants it)
  if (fused_x) rc = rtxb_mxfp8_gemm_glu_mx_fused_x(x, k, qg, sg, h, qh, sh, m, inter, k, inter, stream, status);
  else rc = rtxb_mxfp8_gemm_glu_mx(qx, sx, qg, sg, h, qh, sh, m, inter, k, inter, stream, status);
  if (rc) return rc;
  if (beside && (rc = mxfp8_quantize_impl(w_down, n_out, inter, inter, qd, sd, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY,
                                          stream, true)))
    return rc;
  return rtxb_mxfp8_gemm(qh, sh, qd, sd, y, m, n_out, inter, n_out, RTXB_OUT_BF16, stream, status);
}

int rtxb_sum_parts_f32_to_bf16(const float* parts, int n_parts, int64_t part_stride, int64_t count, void* out_bf16,
                               void* stream) {
  if (!parts || !out_bf16) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (n_parts <= 0 || count <= 0 || part_stride < count) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (!aligned(parts, 16) || !aligned(out_bf16, 16) || part_stride % 4 != 0)
    return fail_msg(RTXB_E_ALIGNMENT, "partials and output must be 16-byte aligned, parts a multiple of 4 floats apart");
  const int64_t ctas = (count / 8 + kReduceThreads - 1) / kReduceThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int grid = static_cast<int>(ctas < 1 ? 1 : (ctas < cap ? ctas : cap));
  sum_parts_f32_to_bf16_kernel<<<grid, kReduceThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      parts, n_parts, part_stride, count, static_cast<__nv_bfloat16*>(out_bf16));
  RTXB_CHECK_LAUNCH("sum_parts_f32_to_bf16_kernel");
  return RTXB_OK;
}

int rtxb_peer_barrier(void* const* rank_flags, int world, int rank, int* epoch_counter, int64_t limit_ns,
                      void* stream, int* status) {
  if (!rank_flags || world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "between 1 and 8 ranks, rank inside the group");
  if (!epoch_counter || !aligned(epoch_counter, 4)) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null epoch counter");
  if (limit_ns < 1000000 || limit_ns > 2000000000ll)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "limit between 1 ms and 2 s");
  PeerFlags flags = {};
  for (int t = 0; t < world; ++t) {
    if (!rank_flags[t] || !aligned(rank_flags[t], 4)) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null or unaligned flag array");
    flags.rank_flags[t] = static_cast<int*>(rank_flags[t]);
  }
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, rank, epoch_counter,
                                                                       static_cast<uint64_t>(limit_ns), status);
  RTXB_CHECK_LAUNCH("peer_barrier_kernel");
  return RTXB_OK;
}

int rtxb_selftest_wait_timeout(int64_t limit_ns, void* stream, int* status, unsigned long long* waited_ns) {
  if (!status) return fail_msg(RTXB_E_INVALID_ARGUMENT, "the self-test reports through the status word");
  if (limit_ns < 1000000 || limit_ns > 2000000000ll)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "limit between 1 ms and 2 s");
  wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t>(limit_ns), status, waited_ns);
  RTXB_CHECK_LAUNCH("wait_selftest_kernel");
  return RTXB_OK;
}

size_t rtxb_mxfp8_backward_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  Carver c(nullptr);
  const int64_t np = round_up(n, 32), mp = round_up(m, 32);
  c.take(m * np);  c.take(rtxb_mxfp8_scale_bytes(m, n, RTXB_SCALE_MMA128));   // dY rows
  c.take(k * np);  c.take(rtxb_mxfp8_scale_bytes(k, n, RTXB_SCALE_MMA128));   // W^T
  c.take(n * mp);  c.take(rtxb_mxfp8_scale_bytes(n, m, RTXB_SCALE_MMA128));   // dY^T
  c.take(k * mp);  c.take(rtxb_mxfp8_scale_bytes(k, m, RTXB_SCALE_MMA128));   // X^T
  return c.off;
}

int rtxb_mxfp8_linear_bwd(const void* dy, const void* x, const void* w, void* dx, void* dw, int dw_dtype, int64_t m,
                          int64_t n, int64_t k, void* workspace, size_t workspace_bytes, void* stream, int* status) {
  if (!workspace || workspace_bytes < rtxb_mxfp8_backward_workspace_bytes(m, n, k))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_mxfp8_linear_bwd");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  if (!dy) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null dy");
  Carver c(workspace);
  const int64_t np = round_up(n, 32), mp = round_up(m, 32);
  uint8_t* qa = c.take(m * np);  uint8_t* sa = c.take(rtxb_mxfp8_scale_bytes(m, n, RTXB_SCALE_MMA128));
  uint8_t* qb = c.take(k * np);  uint8_t* sb = c.take(rtxb_mxfp8_scale_bytes(k, n, RTXB_SCALE_MMA128));
  uint8_t* qc = c.take(n * mp);  uint8_t* sc = c.take(rtxb_mxfp8_scale_bytes(n, m, RTXB_SCALE_MMA128));
  uint8_t* qd = c.take(k * mp);  uint8_t* sd = c.take(rtxb_mxfp8_scale_bytes(k, m, RTXB_SCALE_MMA128));
  int rc;
  const bool shared_dy = dx && dw;   // both products: dY is read once for its row and its transposed quantization
  if (shared_dy &&
      (rc = rtxb_mxfp8_quantize_dual(dy, m, n, n, qa, sa, qc, sc, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
    return rc;
  if (dx) {
    if (!w) return fail_msg(RTXB_E_INVALID_ARGUMENT, "dx needs w");
    // A = dY [M, N] blocks along N; B = W^T as [K rows, N] blocks along N (W stored [N, K])
    if (!shared_dy &&
        (rc = rtxb_mxfp8_quantize(dy, m, n, n, qa, sa, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
      return rc;
    if ((rc = rtxb_mxfp8_quantize_transposed(w, k, n, k, qb, sb, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
      return rc;
    if ((rc = rtxb_mxfp8_gemm(qa, sa, qb, sb, dx, m, k, n, k, RTXB_OUT_BF16, stream, status))) return rc;
  }
  if (dw) {
    if (!x) return fail_msg(RTXB_E_INVALID_ARGUMENT, "dw needs x");
    // A = dY^T as [N rows, M] blocks along M (dY stored [M, N]); B = X^T as [K rows, M] (X stored [M, K])
    if (!shared_dy &&
        (rc = rtxb_mxfp8_quantize_transposed(dy, n, m, n, qc, sc, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
      return rc;
    if ((rc = rtxb_mxfp8_quantize_transposed(x, k, m, k, qd, sd, RTXB_SCALE_MMA128, RTXB_ROUND_INFINITY, stream)))
      return rc;
    if ((rc = rtxb_mxfp8_gemm(qc, sc, qd, sd, dw, n, k, m, k, dw_dtype, stream, status))) return rc;
  }
  return RTXB_OK;
}

namespace {
// |max| over the tensor, then the outer-scale rule; kernel_form selects how the reference forms
// amax / 2688 (see nvfp4_scale_from_amax_bits)
int tensor_scale_impl(const void* src, int64_t rows, int64_t k, int64_t ld, int mode, void* amax_scratch,
                      float* scale_out, const float* other_scale, float* out_scale, void* stream, bool kernel_form) {
  if (!src || !amax_scratch || !scale_out) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (mode != RTXB_TENSOR_SCALE_EXACT && mode != RTXB_TENSOR_SCALE_POWER2)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown tensor scale mode");
  if ((out_scale == nullptr) != (other_scale == nullptr))
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "other_scale and out_scale go together");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, 4, s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(amax)");
  const int64_t work = rows * k / 8 / 256 / 4 + 1;
  const int grid = static_cast<int>(work < sm_count() * 8 ? work : sm_count() * 8);
  amax_bf16_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), rows, k, ld,
                                        static_cast<uint32_t*>(amax_scratch));
  RTXB_CHECK_LAUNCH("amax_bf16_kernel");
  nvfp4_tensor_scale_kernel<<<1, 1, 0, s>>>(static_cast<const uint32_t*>(amax_scratch), mode, scale_out, other_scale,
                                            out_scale, kernel_form);
  RTXB_CHECK_LAUNCH("nvfp4_tensor_scale_kernel");
  return RTXB_OK;
}
}  // namespace

int rtxb_nvfp4_tensor_scale(const void* src, int64_t rows, int64_t k, int64_t ld, int mode, void* amax_scratch,
                            float* scale_out, const float* other_scale, float* out_scale, void* stream) {
  return tensor_scale_impl(src, rows, k, ld, mode, amax_scratch, scale_out, other_scale, out_scale, stream, false);
}

int rtxb_nvfp4_quantize(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales, int scale_layout,
                        const float* tensor_scale, void* stream) {
  if (!src || !q || !scales) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (rows > INT32_MAX || k > INT32_MAX - 512) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q, 16)) return fail_msg(RTXB_E_ALIGNMENT, "q must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantNvParams p;
  p.src = static_cast<const __nv_bfloat16*>(src);
  p.q = static_cast<uint8_t*>(q);
  p.scales = static_cast<uint8_t*>(scales);
  p.tensor_scale = tensor_scale;
  p.region_scales = nullptr;
  p.region_rows = 0;
  p.rows = static_cast<int>(rows);
  p.k = static_cast<int>(k);
  p.kp = static_cast<int>(round_up(k, 32));
  p.ld = ld;
  p.nb = p.kp / 16;
  p.sf_chunks = static_cast<int>(round_up((p.nb + 3) / 4, 4));
  p.layout = scale_layout;
  const int64_t tiles = ((rows + 127) / 128) * ((p.kp + 255) / 256);
  quant_nvfp4_rows_kernel<<<quant_grid(tiles, 4), kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  RTXB_CHECK_LAUNCH("quant_nvfp4_rows_kernel");
  return RTXB_OK;
}

int rtxb_nvfp4_quantize_dynamic(const void* src, int64_t rows, int64_t k, int64_t ld, int mode, void* q, void* scales,
                                int scale_layout, float* scale_out, const float* other_scale, float* out_scale,
                                void* amax_scratch, void* stream) {
  if (!src || !q || !scales || !scale_out || !amax_scratch) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (mode != RTXB_TENSOR_SCALE_EXACT && mode != RTXB_TENSOR_SCALE_POWER2)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown tensor scale mode");
  if ((out_scale == nullptr) != (other_scale == nullptr))
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "other_scale and out_scale go together");
  if (!aligned(amax_scratch, 4)) return fail_msg(RTXB_E_ALIGNMENT, "amax_scratch must be 4-byte aligned");
  const int64_t kp = round_up(k, 32);
  const int64_t tiles = ((rows + 127) / 128) * ((kp + 255) / 256);
  if (tiles > kDynamicMaxPartials) {
    // large tensors: the grid-wide |max| pass, the finalize launch and the quantizer
    int rc = rtxb_nvfp4_tensor_scale(src, rows, k, ld, mode, amax_scratch, scale_out, other_scale, out_scale, stream);
    if (rc) return rc;
    return rtxb_nvfp4_quantize(src, rows, k, ld, q, scales, scale_layout, scale_out, stream);
  }
  if (rows > INT32_MAX || k > INT32_MAX - 512) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q, 16)) return fail_msg(RTXB_E_ALIGNMENT, "q must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantNvDynamicParams dp;
  dp.q.src = static_cast<const __nv_bfloat16*>(src);
  dp.q.q = static_cast<uint8_t*>(q);
  dp.q.scales = static_cast<uint8_t*>(scales);
  dp.q.tensor_scale = nullptr;
  dp.q.region_scales = nullptr;
  dp.q.region_rows = 0;
  dp.q.rows = static_cast<int>(rows);
  dp.q.k = static_cast<int>(k);
  dp.q.kp = static_cast<int>(kp);
  dp.q.ld = ld;
  dp.q.nb = dp.q.kp / 16;
  dp.q.sf_chunks = static_cast<int>(round_up((dp.q.nb + 3) / 4, 4));
  dp.q.layout = scale_layout;
  dp.mode = mode;
  dp.partials = static_cast<const uint32_t*>(amax_scratch);
  dp.n_partials = static_cast<int>(tiles);
  dp.scale_out = scale_out;
  dp.other_scale = other_scale;
  dp.out_scale = out_scale;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = launch_dependent(amax_partials_kernel, static_cast<int>(tiles), kQuantThreads, 0, s, true, dp.q,
                                   static_cast<uint32_t*>(amax_scratch));
  if (e != cudaSuccess) return fail_cuda(e, "amax_partials_kernel launch");
  e = launch_dependent(quant_nvfp4_dynamic_kernel, static_cast<int>(tiles), kQuantThreads, 0, s, true, dp);
  if (e != cudaSuccess) return fail_cuda(e, "quant_nvfp4_dynamic_kernel launch");
  return RTXB_OK;
}

int rtxb_nvfp4_quantize_delayed(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                                int scale_layout, const float* history, float* next_history, int history_len,
                                int window_max, int mode, float* scale_out, const float* other_scale, float* out_scale,
                                void* stream) {
  if (!src || !q || !scales || !history || !next_history || !scale_out)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (history_len != 1 && history_len != 4 && history_len != 16 && history_len != 64)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "amax history must have 1, 4, 16 or 64 values");
  if (history == next_history) return fail_msg(RTXB_E_INVALID_ARGUMENT, "amax history generations must not alias");
  if (mode != RTXB_TENSOR_SCALE_EXACT && mode != RTXB_TENSOR_SCALE_POWER2)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown tensor scale mode");
  if ((out_scale == nullptr) != (other_scale == nullptr))
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "other_scale and out_scale go together");
  if (rows > INT32_MAX || k > INT32_MAX - 512) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q, 16)) return fail_msg(RTXB_E_ALIGNMENT, "q must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(next_history, 0, 4, s);   // the observed |max| is accumulated with an atomic max
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(next history)");
  QuantNvDelayedParams dp;
  dp.q.src = static_cast<const __nv_bfloat16*>(src);
  dp.q.q = static_cast<uint8_t*>(q);
  dp.q.scales = static_cast<uint8_t*>(scales);
  dp.q.tensor_scale = nullptr;
  dp.q.region_scales = nullptr;
  dp.q.region_rows = 0;
  dp.q.rows = static_cast<int>(rows);
  dp.q.k = static_cast<int>(k);
  dp.q.kp = static_cast<int>(round_up(k, 32));
  dp.q.ld = ld;
  dp.q.nb = dp.q.kp / 16;
  dp.q.sf_chunks = static_cast<int>(round_up((dp.q.nb + 3) / 4, 4));
  dp.q.layout = scale_layout;
  dp.history = history;
  dp.next_history = next_history;
  dp.history_len = history_len;
  dp.entries = window_max ? history_len : 1;
  dp.mode = mode;
  dp.scale_out = scale_out;
  dp.other_scale = other_scale;
  dp.out_scale = out_scale;
  const int64_t tiles = ((rows + 127) / 128) * ((dp.q.kp + 255) / 256);
  quant_nvfp4_delayed_kernel<<<quant_grid(tiles, 4), kQuantThreads, 0, s>>>(dp);
  RTXB_CHECK_LAUNCH("quant_nvfp4_delayed_kernel");
  return RTXB_OK;
}

int rtxb_nvfp4_region_scales(const void* src, int64_t rows, int64_t k, int64_t ld, int64_t region_rows, int mode,
                             void* amax_scratch, float* scales_out, void* stream) {
  if (!src || !scales_out) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (region_rows <= 0 || rows % region_rows) return fail_msg(RTXB_E_INVALID_ARGUMENT, "region_rows must divide rows");
  if (mode != RTXB_TENSOR_SCALE_EXACT && mode != RTXB_TENSOR_SCALE_POWER2)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown tensor scale mode");
  if (rows > INT32_MAX || k > INT32_MAX) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (region_rows == rows) {
    // one region = the tensor: the grid-wide reduction
    if (!amax_scratch) return fail_msg(RTXB_E_INVALID_ARGUMENT, "amax_scratch is needed for a single region");
    return tensor_scale_impl(src, rows, k, ld, mode, amax_scratch, scales_out, nullptr, nullptr, stream, true);
  }
  const int64_t regions = rows / region_rows;
  if (region_rows * k * 2 >= 32768) {
    // a whole CTA per region: enough bytes per region to keep 256 threads' loads in flight
    const int grid = static_cast<int>(regions < sm_count() * 8 ? regions : sm_count() * 8);
    amax_regions_cta_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<int>(rows), static_cast<int>(k), ld,
        static_cast<int>(region_rows), mode, scales_out);
    RTXB_CHECK_LAUNCH("amax_regions_cta_kernel");
    return RTXB_OK;
  }
  const int64_t ctas = (regions + 7) / 8;   // small regions: one warp per region, eight warps per CTA
  const int grid = static_cast<int>(ctas < sm_count() * 8 ? ctas : sm_count() * 8);
  amax_regions_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<int>(rows), static_cast<int>(k), ld,
      static_cast<int>(region_rows), mode, scales_out);
  RTXB_CHECK_LAUNCH("amax_regions_kernel");
  return RTXB_OK;
}

int rtxb_nvfp4_quantize_regions(const void* src, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                                int scale_layout, const float* region_scales, int64_t region_rows, void* stream) {
  if (!src || !q || !scales || !region_scales) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (rows <= 0 || k <= 0 || ld < k) return fail_msg(RTXB_E_INVALID_ARGUMENT, "bad shape");
  if (region_rows <= 0 || rows % region_rows) return fail_msg(RTXB_E_INVALID_ARGUMENT, "region_rows must divide rows");
  if (rows > INT32_MAX || k > INT32_MAX - 512) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (scale_layout == RTXB_SCALE_MMA64) return fail_msg(RTXB_E_UNSUPPORTED, "mma64 scale layout is SM120-only");
  if (scale_layout != RTXB_SCALE_ROW_MAJOR && scale_layout != RTXB_SCALE_MMA128)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown scale layout");
  if (!aligned(q, 16)) return fail_msg(RTXB_E_ALIGNMENT, "q must be 16-byte aligned");
  if (scale_layout == RTXB_SCALE_MMA128 && !aligned(scales, 16))
    return fail_msg(RTXB_E_ALIGNMENT, "mma128 scale tiles must be 16-byte aligned");
  QuantNvParams p;
  p.src = static_cast<const __nv_bfloat16*>(src);
  p.q = static_cast<uint8_t*>(q);
  p.scales = static_cast<uint8_t*>(scales);
  p.tensor_scale = nullptr;
  p.region_scales = region_scales;
  p.region_rows = static_cast<int>(region_rows);
  p.rows = static_cast<int>(rows);
  p.k = static_cast<int>(k);
  p.kp = static_cast<int>(round_up(k, 32));
  p.ld = ld;
  p.nb = p.kp / 16;
  p.sf_chunks = static_cast<int>(round_up((p.nb + 3) / 4, 4));
  p.layout = scale_layout;
  const int64_t tiles = ((rows + 127) / 128) * ((p.kp + 255) / 256);
  quant_nvfp4_regions_kernel<<<quant_grid(tiles, 4), kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  RTXB_CHECK_LAUNCH("quant_nvfp4_regions_kernel");
  return RTXB_OK;
}

int rtxb_nvfp4_gemm_regions(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m,
                            int64_t n, int64_t k, int64_t ldo, const float* x_region_scales, int64_t x_region_rows,
                            const float* w_region_scales, int64_t w_region_rows, void* stream, int* status) {
  int rc = check_gemm_args(qa, sa, qb, sb, out, m, n, k, ldo, n, 2);
  if (rc) return rc;
  if (!x_region_scales || !w_region_scales) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null region scales");
  if (x_region_rows <= 0 || m % x_region_rows || w_region_rows <= 0 || n % w_region_rows)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "region rows must divide the operand's rows");
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = round_up((kp / 16 + 3) / 4, 4);
  const RegionScales rs{x_region_scales, w_region_scales, static_cast<int>(x_region_rows),
                        static_cast<int>(w_region_rows)};
  return launch_gemm<kKindNvfp4, kEpiRegionBf16>(qa, sa, qb, sb, out, m, n, kp / 2, chunks, ldo, n, 0, nullptr,
                                                 static_cast<cudaStream_t>(stream), status, nullptr, nullptr, false,
                                                 &rs);
}

int rtxb_nvfp4_gemm(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n,
                    int64_t k, int64_t ldo, int out_dtype, const float* output_scale, void* stream, int* status) {
  if (out_dtype != RTXB_OUT_BF16 && out_dtype != RTXB_OUT_F32)
    return fail_msg(RTXB_E_INVALID_ARGUMENT, "unknown output dtype");
  int rc = check_gemm_args(qa, sa, qb, sb, out, m, n, k, ldo, n, out_dtype == RTXB_OUT_BF16 ? 2 : 4);
  if (rc) return rc;
  const int64_t kp = round_up(k, 32);
  const int64_t chunks = round_up((kp / 16 + 3) / 4, 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == RTXB_OUT_BF16)
    return launch_gemm<kKindNvfp4, kEpiBf16>(qa, sa, qb, sb, out, m, n, kp / 2, chunks, ldo, n, 0, output_scale, s, status);
  return launch_gemm<kKindNvfp4, kEpiF32>(qa, sa, qb, sb, out, m, n, kp / 2, chunks, ldo, n, 0, output_scale, s, status);
}

size_t rtxb_nvfp4_linear_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  Carver c(nullptr);
  const int64_t kp = round_up(k, 32);
  c.take(256);
  c.take(m * kp / 2);
  c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  c.take(n * kp / 2);
  c.take(rtxb_nvfp4_scale_bytes(n, k, RTXB_SCALE_MMA128));
  return c.off;
}

int rtxb_nvfp4_linear_fwd(const void* x, const void* w, void* out, int64_t m, int64_t n, int64_t k, int scale_mode,
                          void* workspace, size_t workspace_bytes, void* stream, int* status) {
  if (!workspace || workspace_bytes < rtxb_nvfp4_linear_workspace_bytes(m, n, k))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_nvfp4_linear_fwd");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  Carver c(workspace);
  const int64_t kp = round_up(k, 32);
  uint8_t* scal = c.take(256);
  uint8_t* qx = c.take(m * kp / 2);
  uint8_t* sx = c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  uint8_t* qw = c.take(n * kp / 2);
  uint8_t* sw = c.take(rtxb_nvfp4_scale_bytes(n, k, RTXB_SCALE_MMA128));
  // scalar block: [0] amax x, [4] amax w, [16] x scale, [20] w scale, [24] output scale
  float* x_scale = reinterpret_cast<float*>(scal + 16);
  float* w_scale = reinterpret_cast<float*>(scal + 20);
  float* o_scale = reinterpret_cast<float*>(scal + 24);
  int rc;
  if ((rc = rtxb_nvfp4_tensor_scale(x, m, k, k, scale_mode, scal, x_scale, nullptr, nullptr, stream))) return rc;
  if ((rc = rtxb_nvfp4_tensor_scale(w, n, k, k, scale_mode, scal + 4, w_scale, x_scale, o_scale, stream))) return rc;
  if ((rc = rtxb_nvfp4_quantize(x, m, k, k, qx, sx, RTXB_SCALE_MMA128, x_scale, stream))) return rc;
  if ((rc = rtxb_nvfp4_quantize(w, n, k, k, qw, sw, RTXB_SCALE_MMA128, w_scale, stream))) return rc;
  return rtxb_nvfp4_gemm(qx, sx, qw, sw, out, m, n, k, n, RTXB_OUT_BF16, o_scale, stream, status);
}

size_t rtxb_nvfp4_linear_prequant_w_workspace_bytes(int64_t m, int64_t k) {
  Carver c(nullptr);
  const int64_t kp = round_up(k, 32);
  c.take(512);
  c.take(m * kp / 2);
  c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  return c.off;
}

int rtxb_nvfp4_linear_fwd_prequant_w(const void* x, const void* qw, const void* sw, const float* w_scale, void* out,
                                     int64_t m, int64_t n, int64_t k, int scale_mode, void* workspace,
                                     size_t workspace_bytes, void* stream, int* status) {
  if (!w_scale) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null weight scale");
  if (!workspace || workspace_bytes < rtxb_nvfp4_linear_prequant_w_workspace_bytes(m, k))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_nvfp4_linear_fwd_prequant_w");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  if (!x || !qw || !sw || !out) return fail_msg(RTXB_E_INVALID_ARGUMENT, "null operand");
  if (m <= 0 || n <= 0 || k <= 0) return fail_msg(RTXB_E_INVALID_ARGUMENT, "m, n, k must be positive");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX - 512) return fail_msg(RTXB_E_UNSUPPORTED, "dimension exceeds int32");
  if (!aligned(sw, 16)) return fail_msg(RTXB_E_ALIGNMENT, "scale tiles must be 16-byte aligned");
  if (!aligned(out, 2)) return fail_msg(RTXB_E_ALIGNMENT, "output pointer is not element aligned");
  int rc;
  Carver c(workspace);
  const int64_t kp = round_up(k, 32);
  uint8_t* scal = c.take(512);
  uint8_t* qx = c.take(m * kp / 2);
  uint8_t* sx = c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  // scalar block: [0, 256) |max| partials, [256] x scale, [264] output scale
  float* x_scale = reinterpret_cast<float*>(scal + 256);
  float* o_scale = reinterpret_cast<float*>(scal + 264);
  if (decode_fused_eligible(x, m, n, k)) {
    // a handful of rows: one kernel quantizes them in every CTA while the weight already streams
    rc = launch_decode_fused(x, qw, sw, w_scale, out, m, n, k, scale_mode, x_scale, static_cast<cudaStream_t>(stream),
                             status);
    return rc;
  }
  rc = rtxb_nvfp4_quantize_dynamic(x, m, k, k, scale_mode, qx, sx, RTXB_SCALE_MMA128, x_scale, w_scale, o_scale, scal,
                                   stream);
  if (rc) return rc;
  // The packed weight was written before the activation quantizer was launched, so the GEMM may
  // start fetching it while that quantizer runs.
  const int64_t chunks = round_up((kp / 16 + 3) / 4, 4);
  return launch_gemm<kKindNvfp4, kEpiBf16>(qx, sx, qw, sw, out, m, n, kp / 2, chunks, n, n, 0, o_scale,
                                           static_cast<cudaStream_t>(stream), status, nullptr, nullptr, true);
}

namespace {
// rows per region actually used: the request when it splits the rows evenly into more than one region,
// else one region over the whole tensor (rtx/fp4.py:89-94)
int64_t effective_region_rows(int64_t rows, int64_t requested) {
  if (requested <= 0 || rows <= requested || rows % requested) return rows;
  return requested;
}
}  // namespace

size_t rtxb_nvfp4_linear_regions_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t x_region_rows,
                                                 int64_t w_region_rows) {
  Carver c(nullptr);
  const int64_t kp = round_up(k, 32);
  c.take(256);
  c.take(4 * (m / effective_region_rows(m, x_region_rows)));
  c.take(4 * (n / effective_region_rows(n, w_region_rows)));
  c.take(m * kp / 2);
  c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  c.take(n * kp / 2);
  c.take(rtxb_nvfp4_scale_bytes(n, k, RTXB_SCALE_MMA128));
  return c.off;
}

int rtxb_nvfp4_linear_fwd_regions(const void* x, const void* w, void* out, int64_t m, int64_t n, int64_t k,
                                  int64_t x_region_rows, int64_t w_region_rows, int scale_mode, void* workspace,
                                  size_t workspace_bytes, void* stream, int* status) {
  if (m <= 0 || n <= 0 || k <= 0) return fail_msg(RTXB_E_INVALID_ARGUMENT, "m, n, k must be positive");
  if (!workspace ||
      workspace_bytes < rtxb_nvfp4_linear_regions_workspace_bytes(m, n, k, x_region_rows, w_region_rows))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_nvfp4_linear_fwd_regions");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  const int64_t rx = effective_region_rows(m, x_region_rows), rw = effective_region_rows(n, w_region_rows);
  Carver c(workspace);
  const int64_t kp = round_up(k, 32);
  uint8_t* scal = c.take(256);
  float* xs = reinterpret_cast<float*>(c.take(4 * (m / rx)));
  float* wsc = reinterpret_cast<float*>(c.take(4 * (n / rw)));
  uint8_t* qx = c.take(m * kp / 2);
  uint8_t* sx = c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  uint8_t* qw = c.take(n * kp / 2);
  uint8_t* sw = c.take(rtxb_nvfp4_scale_bytes(n, k, RTXB_SCALE_MMA128));
  int rc;
  const bool small_regions = rx != m && rw != n && rx * k * 2 < 32768 && rw * k * 2 < 32768 && m <= INT32_MAX &&
                             n <= INT32_MAX && k <= INT32_MAX - 512 && x && w &&
                             (scale_mode == RTXB_TENSOR_SCALE_EXACT || scale_mode == RTXB_TENSOR_SCALE_POWER2);
  if (small_regions) {
    // Layers whose regions are small (one warp per region): both operands' region scales in one launch, both
    // quantizations in a second one (a programmatic dependent of the first), the GEMM behind them as a dependent
    // too: three launches instead of five.  On such layers the launches, not the work, are the time.
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const RegionScaleJob ja{static_cast<const __nv_bfloat16*>(x), xs, static_cast<int>(m), static_cast<int>(rx), k};
    const RegionScaleJob jb{static_cast<const __nv_bfloat16*>(w), wsc, static_cast<int>(n), static_cast<int>(rw), k};
    const int64_t regions = m / rx + n / rw;
    const int64_t ctas = (regions + 7) / 8;
    amax_regions2_kernel<<<static_cast<int>(ctas < sm_count() * 8 ? ctas : sm_count() * 8), 256, 0, st>>>(
        ja, jb, static_cast<int>(k), scale_mode);
    RTXB_CHECK_LAUNCH("amax_regions2_kernel");
    QuantNvParams p[2];
    const void* src[2] = {x, w};
    uint8_t* q[2] = {qx, qw};
    uint8_t* sc[2] = {sx, sw};
    const float* rs[2] = {xs, wsc};
    const int64_t rows[2] = {m, n}, rr[2] = {rx, rw};
    int64_t tiles = 0;
    for (int i = 0; i < 2; ++i) {
      p[i] = QuantNvParams{};
      p[i].src = static_cast<const __nv_bfloat16*>(src[i]);
      p[i].q = q[i];
      p[i].scales = sc[i];
      p[i].tensor_scale = nullptr;
      p[i].region_scales = rs[i];
      p[i].region_rows = static_cast<int>(rr[i]);
      p[i].rows = static_cast<int>(rows[i]);
      p[i].k = static_cast<int>(k);
      p[i].kp = static_cast<int>(kp);
      p[i].ld = k;
      p[i].nb = p[i].kp / 16;
      p[i].sf_chunks = static_cast<int>(round_up((p[i].nb + 3) / 4, 4));
      p[i].layout = RTXB_SCALE_MMA128;
      tiles += ((rows[i] + 127) / 128) * ((p[i].kp + 255) / 256);
    }
    cudaError_t le = launch_dependent(quant_nvfp4_regions2_kernel, quant_grid(tiles, 4), kQuantThreads, 0, st, true, p[0],
                                      p[1]);
    if (le != cudaSuccess) return fail_cuda(le, "quant_nvfp4_regions2_kernel launch");
    if ((rc = check_gemm_args(qx, sx, qw, sw, out, m, n, k, n, n, 2))) return rc;
    const RegionScales rsc{xs, wsc, static_cast<int>(rx), static_cast<int>(rw)};
    return launch_gemm<kKindNvfp4, kEpiRegionBf16>(qx, sx, qw, sw, out, m, n, kp / 2, round_up((kp / 16 + 3) / 4, 4), n, n, 0,
                                                   nullptr, st, status, nullptr, nullptr, false, &rsc, nullptr, true);
  }
  if ((rc = rtxb_nvfp4_region_scales(x, m, k, k, rx, scale_mode, scal, xs, stream))) return rc;
  if ((rc = rtxb_nvfp4_region_scales(w, n, k, k, rw, scale_mode, scal + 4, wsc, stream))) return rc;
  if ((rc = rtxb_nvfp4_quantize_regions(x, m, k, k, qx, sx, RTXB_SCALE_MMA128, xs, rx, stream))) return rc;
  if ((rc = rtxb_nvfp4_quantize_regions(w, n, k, k, qw, sw, RTXB_SCALE_MMA128, wsc, rw, stream))) return rc;
  return rtxb_nvfp4_gemm_regions(qx, sx, qw, sw, out, m, n, k, n, xs, rx, wsc, rw, stream, status);
}

int rtxb_nvfp4_linear_fwd_delayed(const void* x, const void* w, void* out, int64_t m, int64_t n, int64_t k,
                                  const float* x_history, const float* w_history, float* next_x_history,
                                  float* next_w_history, int history_len, int window_max, int scale_mode,
                                  void* workspace, size_t workspace_bytes, void* stream, int* status) {
  if (m <= 0 || n <= 0 || k <= 0) return fail_msg(RTXB_E_INVALID_ARGUMENT, "m, n, k must be positive");
  if (!workspace || workspace_bytes < rtxb_nvfp4_linear_workspace_bytes(m, n, k))
    return fail_msg(RTXB_E_WORKSPACE, "workspace too small for rtxb_nvfp4_linear_fwd_delayed");
  if (!aligned(workspace, 256)) return fail_msg(RTXB_E_ALIGNMENT, "workspace must be 256-byte aligned");
  Carver c(workspace);
  const int64_t kp = round_up(k, 32);
  uint8_t* scal = c.take(256);
  uint8_t* qx = c.take(m * kp / 2);
  uint8_t* sx = c.take(rtxb_nvfp4_scale_bytes(m, k, RTXB_SCALE_MMA128));
  uint8_t* qw = c.take(n * kp / 2);
  uint8_t* sw = c.take(rtxb_nvfp4_scale_bytes(n, k, RTXB_SCALE_MMA128));
  float* x_scale = reinterpret_cast<float*>(scal + 16);
  float* w_scale = reinterpret_cast<float*>(scal + 20);
  float* o_scale = reinterpret_cast<float*>(scal + 24);
  int rc;
  if ((rc = rtxb_nvfp4_quantize_delayed(x, m, k, k, qx, sx, RTXB_SCALE_MMA128, x_history, next_x_history, history_len,
                                        window_max, scale_mode, x_scale, nullptr, nullptr, stream)))
    return rc;
  if ((rc = rtxb_nvfp4_quantize_delayed(w, n, k, k, qw, sw, RTXB_SCALE_MMA128, w_history, next_w_history, history_len,
                                        window_max, scale_mode, w_scale, x_scale, o_scale, stream)))
    return rc;
  return rtxb_nvfp4_gemm(qx, sx, qw, sw, out, m, n, k, n, RTXB_OUT_BF16, o_scale, stream, status);
}

}  // extern "C"
