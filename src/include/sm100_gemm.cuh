// Persistent tcgen05 GEMM core shared by the plain GEMM (src/ops/gemm_sm100.cu)
// and the fused tensor-parallel kernels (src/tp).  C tile = A[128 x K] · B[BN x K]^T,
// bf16 operands (K-major), fp32 accumulation in TMEM.
//
// Roles inside one CTA of 192 threads:
//   warp 0     TMA producer (tile loads, 128-byte swizzle, STAGES-deep mbarrier ring)
//   warp 1     TMEM allocation + single-thread tcgen05.mma issue + tcgen05.commit
//   warps 2-5  epilogue: tcgen05.ld of one 32-lane quarter each, then Policy::store
// A Policy decides the tile order, may gate the loads of a row block on data that
// another GPU has to deliver first, and owns the epilogue (where a tile goes, what
// is added to it, which flag is raised afterwards):
//
//   struct Policy {
//     int  num_tiles() const;
//     void tile(int idx, int& m_blk, int& n_blk) const;              // idx: position in this rank's tile order
//     const CUtensorMap* a_map(int m_blk, int& row0) const;          // tensor map + first row for the A tile
//     bool gate(int m_blk, volatile int* abort) const;               // producer: wait until row block m_blk may be loaded
//     bool tile_begin(int m_blk, int n_blk, int et, volatile int* abort);   // epilogue threads (et 0..127), before the stores
//     void store(int m_blk, int n_blk, int row, int col0, float (&v)[32]);  // 32 consecutive columns of one row
//     void tile_end(int m_blk, int n_blk, int et);                   // after all 128 epilogue threads stored (barrier done)
//     static constexpr int STAGING; void set_staging(uint8_t*);      // bytes of shared memory the epilogue wants, and where they are
//   };
// Every wait is bounded; see gemm_persistent for the abort protocol.
#pragma once
#include "sm100_ptx.cuh"

namespace sm100 {

constexpr int GEMM_BM = 128, GEMM_BK = 64, GEMM_THREADS = 192;
constexpr unsigned long long kGemmWaitLimitNs = 4000000000ull;   // 4 s

template <int BN, int STAGES, int STAGING = 0>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2, B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;          // epilogue staging tile (policies that store through shared memory)
  static constexpr int BAR_OFF = STAGING_OFF + STAGING;
  static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;          // slack for the 1024-byte alignment of the tiles
};

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Runs the whole persistent loop for this CTA: tiles first_tile, first_tile + stride, ...
// `s_abort` is a CTA-wide flag in shared memory (zeroed by the caller before the first barrier).
// On a wait that runs out: status word set (1 producer, 2/3 MMA issuer, 4 epilogue, 5 policy gate),
// every role leaves its loop, in-flight copies get time to land, TMEM is released.
template <int BN, int STAGES, class Policy>
__device__ __forceinline__ void gemm_persistent(uint8_t* smem_raw, const CUtensorMap* tmap_b, Policy& pol, int K, int first_tile, int tile_stride,
                                                int* status, volatile int* s_abort) {
  typedef GemmSmem<BN, STAGES, Policy::STAGING> L;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  pol.set_staging(smem + L::STAGING_OFF);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = pol.num_tiles(), num_kb = K / GEMM_BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 128); }
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) tma_prefetch_desc(tmap_b);
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int t = first_tile; t < num_tiles && !*s_abort; t += tile_stride) {
        int m_blk, n_blk; pol.tile(t, m_blk, n_blk);
        if (!pol.gate(m_blk, s_abort)) { *s_abort = 1; atomicExch(status, 5); break; }
        int row0; const CUtensorMap* ta = pol.a_map(m_blk, row0);
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, s_abort, kGemmWaitLimitNs)) { atomicExch(status, 1); ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES; uint8_t* sb = sa + L::A_BYTES;
          mbar_arrive_expect_tx(&full[stage], L::STAGE_BYTES);
          tma_load_2d(sa, ta, kb * GEMM_BK, row0, &full[stage]);
          tma_load_2d(sb, tmap_b, kb * GEMM_BK, n_blk * BN, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN);
      int stage = 0; uint32_t phase = 0; int local = 0;
      for (int t = first_tile; t < num_tiles && !*s_abort; t += tile_stride, local++) {
        const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, s_abort, kGemmWaitLimitNs)) { atomicExch(status, 2); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full[stage], phase, s_abort, kGemmWaitLimitNs)) { atomicExch(status, 3); ok = false; break; }
          tc_fence_after();
          const uint8_t* sa = smem + stage * L::STAGE_BYTES; const uint8_t* sb = sa + L::A_BYTES;
          const uint64_t da = make_smem_desc_k128(sa), db = make_smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; k++) umma_f16(d_tmem, desc_advance(da, k * 32), desc_advance(db, k * 32), idesc, (kb | k) != 0);
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;                 // the TMEM lane quarter this warp may read
    const int et = (warp - 2) * 32 + lane;        // 0..127
    int local = 0;
    for (int t = first_tile; t < num_tiles; t += tile_stride, local++) {
      int m_blk, n_blk; pol.tile(t, m_blk, n_blk);
      const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, s_abort, kGemmWaitLimitNs)) { atomicExch(status, 4); break; }
      tc_fence_after();
      if (!pol.tile_begin(m_blk, n_blk, et, s_abort)) { *s_abort = 1; atomicExch(status, 6); break; }
      const int row = quarter * 32 + lane;        // row inside the tile == TMEM lane
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
        pol.store(m_blk, n_blk, row, c * 32, v);
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);              // accumulator may be overwritten
      epilogue_barrier();                         // all 128 threads stored this tile
      pol.tile_end(m_blk, n_blk, et);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    unsigned long long t0 = gtime_ns();
    while (gtime_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// 32 fp32 values -> 32 bf16 (64 bytes) at p
__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16* p, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; j++) o2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
    *reinterpret_cast<uint4*>(p + i) = o;
  }
}
// v += 32 bf16 read from p with L1 bypass (data another GPU wrote)
__device__ __forceinline__ void add_row32_bf16_volatile(const __nv_bfloat16* p, float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    uint4 b;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + i) : "memory");
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int j = 0; j < 4; j++) { float2 f = __bfloat1622float2(b2[j]); v[i + 2 * j] += f.x; v[i + 2 * j + 1] += f.y; }
  }
}

}  // namespace sm100
