// Shared device helpers for the sm_100a kernels: PTX wrappers (mbarrier, TMA,
// tcgen05/TMEM), descriptor builders and the scalar numerics of the MXFP8 /
// NVFP4 encoders.  Everything here is header-only and has no host state.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rtxb {

// ---------------------------------------------------------------------------
// status word written by kernels (0 = ok).  Kernels never trap: a wait that
// runs out records where it gave up and the CTA leaves through its normal
// teardown (TMEM freed), so the context stays usable.
// ---------------------------------------------------------------------------
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusWaitProducer = 1,   // TMA producer gave up waiting for a free stage
  kStatusWaitMma = 2,        // MMA issuer gave up waiting for operands / TMEM
  kStatusWaitEpilogue = 3,   // epilogue gave up waiting for accumulators
  kStatusWaitQuant = 4,      // quantizer warps gave up waiting for a BF16 tile
  kStatusWaitSelfTest = 5,   // the wait self-test's barrier (which nothing ever completes) ran out, as it must
  kStatusWaitPeer = 6,       // node barrier: another rank's flag never arrived
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// true in exactly one lane of a fully active warp (always the same lane)
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrive on a barrier named by a shared::cluster address (own CTA or a peer of the cluster)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when ~kWaitLimitNs elapsed without the phase
// completing (or when another role already raised the CTA's abort flag); the
// caller then records a status and leaves its loop.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t start = 0;
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0x3FF) == 0) {
      if (*abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// TMA (no cluster multicast anywhere: every CTA fetches its own tiles)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0,
                                            int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// 3-D tile: used with a [K / 128][rows][128 bytes] view of a payload so that one instruction fetches
// several consecutive K steps of a row block (each lands as its own 128-byte-swizzled tile)
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0,
                                            int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on `bar` once every tcgen05 op issued earlier by this thread is done.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into all
// four 32-lane quadrants (the scale-factor staging copy).
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8f6f4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tc_mma_mxf4nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// One warp reads its 32 TMEM lanes x 32 consecutive 32-bit columns: thread t
// receives row (lane quadrant base + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// CTA pairs (cluster of two, tcgen05 cta_group::2).  No TMA multicast: each CTA of the
// pair fetches its own half of the operands; what the pair shares is read by the MMA from
// both CTAs' shared memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Programmatic dependent launch.  `griddep_wait` returns once every grid this one depends on has
// completed and its writes are visible (at once when the launch carried no such dependency);
// `griddep_launch_dependents` lets a dependent grid start its own prologue early.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// TMA tile load whose completion is signalled on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// commit that arrives on the barrier at the same shared-memory offset in every CTA of `cta_mask`
// (the arrival is multicast, not a load)
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
__device__ __forceinline__ void tc_cp_32x128b_warpx4_pair(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8f6f4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                     uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tc_mma_mxf4nvf4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                     uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// Shared-memory matrix descriptor, K-major operand tile stored as rows of 128
// bytes with the 128-byte swizzle (what a SWIZZLE_128B TMA box writes).  Eight
// rows form one 1024-byte swizzle atom, so the stride between row groups is
// 1024 bytes; the leading-dimension offset is unused for swizzled K-major
// tiles.  Fields: start address >> 4 in [0,14), LBO >> 4 in [16,30),
// SBO >> 4 in [32,46), descriptor version 1 in [46,48), layout type in [61,64)
// (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Descriptor of a 32-row x 16-byte unswizzled block (row pitch 16 bytes; eight
// rows = one 128-byte core matrix, so SBO = 128), the source of the
// scale-factor copy above.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

// Block-scaled instruction descriptor (upper word of the 64-bit form):
//  [4,6) B scale id  [7,10) A format  [10,13) B format  [15] A major  [16] B major
//  [17,23) N>>3  [23] scale format (0 = UE4M3, 1 = UE8M0)  [24,29) M>>4  [29,31) A scale id.
// kind::mxf8f6f4 formats: E4M3 = 0.  kind::mxf4nvf4 formats: E2M1 = 1.
__host__ __device__ constexpr uint32_t idesc_block_scaled(uint32_t m, uint32_t n, uint32_t ab_format,
                                                          uint32_t scale_is_ue8m0) {
  return (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | (scale_is_ue8m0 << 23) | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
  return idesc | (a_id << 29) | (b_id << 4);
}

// ---------------------------------------------------------------------------
// MXFP8 / NVFP4 scalar numerics
// ---------------------------------------------------------------------------

// Per-block |max| -> biased E8M0 code and the exact FP32 reciprocal of the
// decode scale.  Integer rule: exponent(amax) - 8, plus one when the mantissa
// exceeds 1.75 (round-to-infinity; skipped for the OCP floor ablation), clamped
// to [-127, 128]; NaN -> 255.
__device__ __forceinline__ uint32_t e8m0_from_amax(float amax, bool round_to_infinity) {
  uint32_t bits = __float_as_uint(amax);
  int exponent = static_cast<int>((bits >> 23) & 0xFF) - 127 - 8;
  if (round_to_infinity && (bits & 0x7FFFFF) > 0x600000) exponent += 1;
  exponent = max(exponent, -127);
  exponent = min(exponent, 128);
  uint32_t biased = static_cast<uint32_t>(exponent + 127);
  if (amax != amax) biased = 255;
  return biased;
}
__device__ __forceinline__ float e8m0_reciprocal(uint32_t biased) {
  uint32_t f = biased == 0 ? 1u : biased;
  uint32_t rbits = (254u - f) << 23;
  if (f == 254u) rbits = 1u << 22;
  if (f == 255u) rbits = 0u;
  return __uint_as_float(rbits);
}
// two FP32 -> two E4M3 codes (lo in bits [0,8), hi in [8,16)), RNE, satfinite
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t out;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(out) : "f"(lo), "f"(hi));
  return out;
}
// two FP32 -> one byte of two E2M1 codes (lo in the low nibble), RNE, satfinite
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t out;
  asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tcvt.u32.u8 %0, b;\n\t}"
      : "=r"(out)
      : "f"(lo), "f"(hi));
  return out;
}
__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
  // exact decode of a non-negative E4M3 scale code (sign bit ignored)
  uint32_t e = (code >> 3) & 0xF, m = code & 0x7;
  if (e == 0) return static_cast<float>(m) * 0.001953125f;  // m * 2^-9
  return __uint_as_float(((e + 120u) << 23) | (m << 20));
}
// NaN-propagating max of magnitudes
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float fmin_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xFFFF0000u); }

// physical byte of (row, block) inside the 128-row scale tiles:
// tiles [row/128][block/4] of 512 bytes, byte (row%32)*16 + ((row/32)%4)*4 + block%4
__host__ __device__ __forceinline__ size_t sf_tile_offset(uint32_t row, uint32_t block, uint32_t chunks_per_row) {
  return (static_cast<size_t>(row >> 7) * chunks_per_row + (block >> 2)) * 512 + (row & 31) * 16 +
         ((row >> 5) & 3) * 4 + (block & 3);
}

}  // namespace rtxb
