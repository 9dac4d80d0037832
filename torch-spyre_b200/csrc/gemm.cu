// fp16 GEMM / batched GEMM on the 5th-generation tensor cores (tcgen05), operands
// and result as stick images, fp32 accumulation in tensor memory.
//
// Stands in for the reference's mm / bmm / addmm eager wrappers
// (codegen/inputs/spyre_torch_ops.cpp:214-452) and its compiled matmul program
// (torch_spyre/_inductor/lowering.py:25-47, codegen/compute_ops.py:396-824).
//
// Why the stick layout suits the tensor cores.  The image of A[batch, M, K] is
// [K/64][batch][M][64]: a 128-row x 64-k tile is 128 consecutive 128-byte rows,
// which is exactly the K-major, 128-byte-swizzled shared-memory tile tcgen05.mma
// consumes, so one 4-D TMA box fetches it.  B[batch, K, N] has image
// [N/64][batch][K][64]: a 64-k x 64-n box is an "MN-major" swizzled operand block.
// A weight stored as [N, K] (the x @ W^T of a linear layer) is K-major like A.
// C[batch, M, N] has image [N/64][batch][M][64]: an accumulator row slice of 64
// columns is one 128-byte stick.
//
// Kernel shape: persistent, one CTA per SM, tile 128 x 256 x 64, kStages-deep
// TMA->smem ring.  Warp 0 issues TMA, warp 1 issues MMAs, warps 2-9 drain the
// accumulator (TMEM -> registers -> fp16 -> global).  TMEM holds two 128x256 fp32
// accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
// When M > 128 the same roles run on pairs of CTAs (clusters of two, tcgen05
// cta_group::2, 256 x 256 tiles): see gemm_f16_pair_kernel below.
// Every wait is bounded; on a timeout the CTA raises a flag, every role leaves its
// loop, TMEM is released and the host-visible error word is set.
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tma_map.cuh"

namespace tsb {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;               // two per tensor-memory lane quarter, 128 accumulator columns each
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBBytes = BN * BK * 2;          // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;   // epilogue: 32 rows x 128 bytes per warp
constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitLimit = 4000000000ll;  // ~2 s of SM clocks
constexpr double kWideCost = 0.80;              // time of a 256 x 512 pair tile relative to two 256 x 256 ones (measured 0.73-0.83)
constexpr long long kDrainLimit = 200000ll;     // ~0.1 ms: far longer than a TMA copy is in flight

__device__ int g_gemm_error;  // sticky: set when a bounded wait gave up
#ifdef TSB_TUNING
// experiment counters of the tuning build: cycles the leaders' MMA threads spent waiting for
// operands [0] and for a drained accumulator [1], their total loop cycles [2], cycles the
// producers waited for a free stage [3], producer loop cycles [4]
__device__ unsigned long long g_gemm_prof[8];
#define TSB_PROF_DECL long long prof_t0 = 0, prof_a = 0, prof_b = 0; const long long prof_start = clock64(); (void)prof_b;
#define TSB_PROF_BEGIN if (!(P.tune_noload & 8)) prof_t0 = clock64();
#define TSB_PROF_END(acc) if (!(P.tune_noload & 8)) acc += clock64() - prof_t0;
#else
#define TSB_PROF_DECL
#define TSB_PROF_BEGIN
#define TSB_PROF_END(acc)
#endif

struct GemmParams {
  __half* c;
  const __half* bias;   // [N] stick image or null
  const __half* residual;   // image shaped and strided like c, added to the rounded product, or null
  int swiglu;               // 1: stick columns of the product alternate gate / up; c = silu(gate) * up
  uint32_t M, N, K, batch, heads;
  int64_t c_stick_stride, c_head_stride;   // elements
  uint32_t tiles_m, tiles_n, num_tiles, k_blocks;
  uint32_t band_tiles;   // tile columns per band of the tile order (see decode_tile)
#ifdef TSB_TUNING
  int tune_noload;       // experiment: 1 = arm the "full" barriers without issuing the TMA loads, 2 = MMAs alone
  int tune_hint;         // experiment: suspend-time hint (ns) for the epilogue's and the producers' waits
  int tune_collect;      // experiment: 2 = never interleave the two halves (A read from shared memory for every MMA)
  int tune_epi;          // experiment: 1 = epilogue releases without draining, 2 = tensor-memory loads only,
                         // 3 = loads and staging but no global stores
#endif
  int b_kmajor;          // 1: B given as [batch, N, K] (K contiguous)
  int b_batched;         // 0: one B shared by every batch
  // Reduce-scatter epilogue: the rows of the product are owned in equal blocks by `owners`
  // buffers (this GPU's and its peers'), and a tile is added into its owner's buffer with
  // fp16x2 reductions instead of being stored.  owners == 0: plain stores into c.
  uint32_t owners, rows_per_owner;
  uint32_t owner_store;   // 1: plain stores into the owners' buffers (each rank writes a slot of its own) instead of reductions
  __half* c_owner[8];
};

struct Barriers {
  uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Tile order within one (batch, head): bands of kBandTiles tile columns, rows fastest across
// a band, so that the tiles in flight at any time (one per CTA or CTA pair) form a roughly
// square block and share both their A row panels and their B column panels in L2.
__device__ __forceinline__ void decode_tile(const GemmParams& P, uint32_t tile, uint32_t tiles_m,
                                            uint32_t& tm, uint32_t& tn, uint32_t& b, uint32_t& h) {
  const uint32_t per_bh = P.tiles_n * tiles_m;
  const uint32_t bh = tile / per_bh, t = tile - bh * per_bh;
  b = bh % P.batch;
  h = bh / P.batch;
  const uint32_t band = t / (P.band_tiles * tiles_m), r = t - band * (P.band_tiles * tiles_m);
  const uint32_t width = min(P.band_tiles, P.tiles_n - band * P.band_tiles);
  tm = r / width;
  tn = band * P.band_tiles + (r - tm * width);
}

// Adds eight fp16 values to memory (this GPU's or, over NVLink, a peer's) without reading them
// back: a vector reduction at system scope.
__device__ __forceinline__ void red_add_v4(void* p, uint4 v) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// 64 accumulator columns of this warp's 32 rows: tensor memory -> registers (no wait).
__device__ __forceinline__ void load_stick(uint32_t taddr, uint32_t (&r)[2][32]) {
  ptx::tmem_ld_32x32(taddr, r[0]);
  ptx::tmem_ld_32x32(taddr + 32, r[1]);
}

// Registers of one stick (fp32, one row per lane) -> fp16 -> the warp's shared-memory staging block
// (32 rows x 128 bytes, 16-byte chunks XOR-swizzled by row so that neither side has bank
// conflicts) -> global memory with every store instruction covering four whole 128-byte sticks
// instead of 16 bytes of 32 different ones.  `res` holds the residual rows this lane will store
// (fetched by the caller ahead of the tensor-memory wait), already in the store layout.
template <bool RES>
__device__ __forceinline__ void store_stick(const GemmParams& P, const uint32_t (&r)[2][32], uint8_t* stage,
                                            __half* dst, uint32_t row0, uint32_t col, const uint4 (&res)[RES ? 8 : 1],
                                            int lane) {
  const int srow = lane >> 3, piece = lane & 7;
#pragma unroll
  for (int sub = 0; sub < 2; ++sub) {
    Vec8h bv[4];
    if (P.bias) {
#pragma unroll
      for (int v = 0; v < 4; ++v) bv[v].u = ld_global_v4(P.bias + col + sub * 32 + v * 8);
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      Vec8h o;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x0 = __uint_as_float(r[sub][v * 8 + 2 * e]), x1 = __uint_as_float(r[sub][v * 8 + 2 * e + 1]);
        if (P.bias) {
          x0 += __half2float(bv[v].h[2 * e]);
          x1 += __half2float(bv[v].h[2 * e + 1]);
        }
        o.h2[e] = __floats2half2_rn(x0, x1);
      }
      *reinterpret_cast<uint4*>(stage + lane * 128 + (((sub * 4 + v) ^ (lane & 7)) * 16)) = o.u;
    }
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + srow;
    Vec8h v;
    v.u = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((piece ^ (rr & 7)) * 16));
    if (row0 + rr < P.M) {
      if (RES) {   // fp16 sum of the rounded product and the residual: what add(r, mm(a, b)) gives
        Vec8h q;
        q.u = res[RES ? i : 0];
#pragma unroll
        for (int e = 0; e < 4; ++e) v.h2[e] = __hadd2(v.h2[e], q.h2[e]);
      }
#ifdef TSB_TUNING
      if (P.tune_epi == 3) { if (v.u.x == 0x7fff7fffu) st_global_v4(dst, v.u); continue; }
#endif
      if (P.owners && !P.owner_store) red_add_v4(dst + (int64_t)rr * kStickHalfs, v.u);
      else st_global_v4(dst + (int64_t)rr * kStickHalfs, v.u);
    }
  }
  __syncwarp();
}

// Drains one warp's share of an accumulator: 32 rows x 128 columns (two sticks).  A stick's
// residual rows are fetched while its tensor-memory loads are in flight.
// `release` tells the MMA thread that this warp no longer needs the accumulator; it is called as
// soon as the values are in registers wherever the registers allow that (the accumulator is the
// scarce thing: the next tile's MMAs wait for it, the stores can trail behind).
template <bool RES, class Release>
__device__ __forceinline__ void drain_rows(const GemmParams& P, uint32_t taddr, uint8_t* stage,
                                           uint32_t row0, uint32_t col0, uint32_t b, uint32_t h,
                                           int lane, Release release) {
  const uint32_t c_sticks = (P.N + 63) / 64;
  const int srow = lane >> 3, piece = lane & 7;
  const uint32_t stick0 = col0 >> 6;
  if (stick0 >= c_sticks) { release(); return; }   // warp-uniform
  const bool two = stick0 + 1 < c_sticks;
  __half* dst0 = P.c + (int64_t)h * P.c_head_stride + (int64_t)stick0 * P.c_stick_stride +
                 ((int64_t)b * P.M + row0) * kStickHalfs + piece * 8;
  if (P.owners) {   // the warp's 32 rows lie in one owner's block (rows_per_owner is a multiple of 32)
    const uint32_t owner = row0 / P.rows_per_owner;
    if (owner >= P.owners) { release(); return; }
    dst0 = P.c_owner[owner] + (int64_t)stick0 * P.c_stick_stride +
           (int64_t)(row0 - owner * P.rows_per_owner) * kStickHalfs + piece * 8;
  }
  uint4 res[RES ? 8 : 1];
  auto fetch_residual = [&](const __half* dst) {
    if (RES) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + srow;
        res[RES ? i : 0] = make_uint4(0, 0, 0, 0);
        if (row0 + rr < P.M) res[RES ? i : 0] = ld_global_v4(P.residual + (dst - P.c) + (int64_t)rr * kStickHalfs);
      }
    }
  };
  // One stick of accumulator values at a time (320 threads leave 168 registers a thread; holding
  // both sticks to release the accumulator earlier spills and measured slower); the other epilogue
  // warp of the lane quarter works on its own sticks meanwhile.  A stick's residual rows are
  // fetched while its tensor-memory loads are in flight.
  uint32_t r[2][32];
#ifdef TSB_TUNING
  if (P.tune_epi == 1) { release(); return; }
#endif
#pragma unroll 1
  for (int k = 0; k < (two ? 2 : 1); ++k) {
    __half* dst = dst0 + k * P.c_stick_stride;
    load_stick(taddr + k * 64, r);
    fetch_residual(dst);
    ptx::tmem_ld_wait();
    if (k == (two ? 1 : 0)) release();
#ifdef TSB_TUNING
    if (P.tune_epi == 2) continue;
#endif
    store_stick<RES>(P, r, stage, dst, row0, col0 + k * 64, res, lane);
  }
}

// The drain for a gate/up projection pair computed as one product whose stick columns alternate
// gate, up, gate, up: a warp's 128 product columns are one (gate, up) pair of sticks and become one
// output stick silu(gate) * up, with the roundings of the unfused sequence (product -> fp16,
// silu -> fp16, multiply -> fp16).
__device__ __forceinline__ float silu_of(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-x * 1.4426950408889634f));
  return x * __fdividef(1.f, 1.f + e);
}
template <class Release>
__device__ __forceinline__ void drain_rows_swiglu(const GemmParams& P, uint32_t taddr, uint8_t* stage,
                                                  uint32_t row0, uint32_t col0, uint32_t b, uint32_t h,
                                                  int lane, Release release) {
  const uint32_t c_sticks = (P.N / 2 + 63) / 64;
  const int srow = lane >> 3, piece = lane & 7;
  const uint32_t stick = col0 >> 7;
  if (stick >= c_sticks) { release(); return; }   // warp-uniform
  uint32_t g[2][32], u[2][32];
  load_stick(taddr, g);
  load_stick(taddr + 64, u);
  ptx::tmem_ld_wait();
  release();
#pragma unroll
  for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      Vec8h o;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = v * 8 + 2 * e;
        const __half2 g16 = __floats2half2_rn(__uint_as_float(g[sub][i]), __uint_as_float(g[sub][i + 1]));
        const __half2 u16 = __floats2half2_rn(__uint_as_float(u[sub][i]), __uint_as_float(u[sub][i + 1]));
        const float2 gf = __half22float2(g16);
        const __half2 s16 = __floats2half2_rn(silu_of(gf.x), silu_of(gf.y));
        o.h2[e] = __hmul2(s16, u16);
      }
      *reinterpret_cast<uint4*>(stage + lane * 128 + (((sub * 4 + v) ^ (lane & 7)) * 16)) = o.u;
    }
  }
  __syncwarp();
  __half* dst = P.c + (int64_t)h * P.c_head_stride + (int64_t)stick * P.c_stick_stride +
                ((int64_t)b * P.M + row0) * kStickHalfs + piece * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + srow;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((piece ^ (rr & 7)) * 16));
    if (row0 + rr < P.M) st_global_v4(dst + (int64_t)rr * kStickHalfs, v);
  }
  __syncwarp();
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;               // 1024-byte aligned stage ring
  uint8_t* gen_tiles = smem_raw + (tiles - raw);
  uint8_t* staging = gen_tiles + kStages * kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + kStagingBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bars->acc_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[a]), kEpilogueWarps);
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t tile = blockIdx.x; ok && tile < P.num_tiles; tile += gridDim.x) {
        uint32_t tm, tn, b, h;
        decode_tile(P, tile, P.tiles_m, tm, tn, b, h);
        const int bb = P.b_batched ? (int)b : 0;
        for (uint32_t kb = 0; kb < P.k_blocks; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->empty[s]), ph ^ 1, abort_flag,
                                      kWaitLimit)) { ok = false; break; }
          const uint32_t full = ptx::smem_u32(&bars->full[s]);
          ptx::mbar_arrive_expect_tx(full, kStageBytes);
          const uint32_t sa = tiles + s * kStageBytes, sb = sa + kABytes;
          ptx::tma_load_5d(sa, &map_a, full, 0, (int)(tm * BM), (int)b, (int)kb, (int)h);
          if (P.b_kmajor) {
            ptx::tma_load_5d(sb, &map_b, full, 0, (int)(tn * BN), bb, (int)kb, (int)h);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_5d(sb + j * (BK * 128), &map_b, full, 0, (int)(kb * BK), bb,
                               (int)(tn * (BN / 64) + j), (int)h);
          }
        }
      }
      // Let copies still in flight land before the CTA can exit.
      const uint32_t issued = it < (uint32_t)kStages ? it : (uint32_t)kStages;
      for (uint32_t k = 0; k < issued; ++k) {
        const uint32_t j = it - 1 - k, s = j % kStages, ph = (j / kStages) & 1;
        ptx::mbar_wait_bounded(ptx::smem_u32(&bars->full[s]), ph, abort_flag, kWaitLimit);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // One thread feeds the tensor pipe, so its instruction count per 64-k step matters:
      // descriptors are kept as a constant high word plus a low word that only ever gets
      // small offsets added (the address field cannot carry out: shared memory < 256 KiB).
      const uint32_t idesc = ptx::idesc_f16_f32(BM, BN, 0, P.b_kmajor ? 0 : 1);
      const uint64_t da0 = ptx::smem_desc_sw128(tiles, 16, 1024);
      const uint64_t db0 = P.b_kmajor ? ptx::smem_desc_sw128(tiles + kABytes, 16, 1024)
                                      : ptx::smem_desc_sw128(tiles + kABytes, BK * 128, 1024);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      // A and K-major B: 16 k = 32 bytes along the swizzled 128-byte row.  MN-major B: 16 k
      // rows = 2048 bytes; 64-wide n blocks are BK*128 bytes apart (leading offset), 8-row
      // groups 1024 apart.
      const uint32_t b_step = P.b_kmajor ? (32u >> 4) : (2048u >> 4);
      const uint32_t full0 = ptx::smem_u32(&bars->full[0]), empty0 = ptx::smem_u32(&bars->empty[0]);
      uint32_t s = 0, ph = 0, local_tile = 0;
      bool ok = true;
      for (uint32_t tile = blockIdx.x; ok && tile < P.num_tiles; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1, acc_ph = (local_tile >> 1) & 1;
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->acc_empty[acc]), acc_ph ^ 1, abort_flag,
                                    kWaitLimit)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < P.k_blocks; ++kb) {
          if (!ptx::mbar_wait_bounded(full0 + s * 8, ph, abort_flag, kWaitLimit)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t so = s * (kStageBytes >> 4);
          uint32_t a_lo = (uint32_t)da0 + so, b_lo = (uint32_t)db0 + so;
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16) {
            ptx::umma_f16(d_tmem, ((uint64_t)a_hi << 32) | a_lo, ((uint64_t)b_hi << 32) | b_lo, idesc,
                          k16 ? 1u : kb);
            a_lo += 32u >> 4;
            b_lo += b_step;
          }
          ptx::umma_commit(empty0 + s * 8);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (ok) ptx::umma_commit(ptx::smem_u32(&bars->acc_full[acc]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t ch = (uint32_t)(warp - 2) >> 2;   // which 128 columns of the accumulator
    uint8_t* my_stage = staging + (warp - 2) * (32 * 128);
    uint32_t local_tile = 0;
    for (uint32_t tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x, ++local_tile) {
      uint32_t tm, tn, b, h;
      decode_tile(P, tile, P.tiles_m, tm, tn, b, h);
      const uint32_t acc = local_tile & 1, acc_ph = (local_tile >> 1) & 1;
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->acc_full[acc]), acc_ph, abort_flag,
                                  kWaitLimit)) break;
      ptx::tc_fence_after_sync();
      auto release = [&] {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[acc]));
      };
      if (P.swiglu)
        drain_rows_swiglu(P, tmem_base + ((q * 32u) << 16) + acc * BN + ch * 128, my_stage,
                          tm * BM + q * 32, tn * BN + ch * 128, b, h, lane, release);
      else if (P.residual)
        drain_rows<true>(P, tmem_base + ((q * 32u) << 16) + acc * BN + ch * 128, my_stage,
                         tm * BM + q * 32, tn * BN + ch * 128, b, h, lane, release);
      else
        drain_rows<false>(P, tmem_base + ((q * 32u) << 16) + acc * BN + ch * 128, my_stage,
                          tm * BM + q * 32, tn * BN + ch * 128, b, h, lane, release);
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(&g_gemm_error, 1);
}

// ---- the same GEMM on CTA pairs ------------------------------------------------------
// A cluster of two CTAs computes one 256-row tile: tcgen05.mma cta_group::2 multiplies the
// 256 rows of A held by the two CTAs (128 each) by a 256-column B block of which each CTA
// loads only its half (128 columns).  The leader CTA (rank 0) owns the "full" barriers (both
// CTAs' TMA loads count on them) and issues the MMAs; it signals "stage free" and "accumulator
// ready" to both CTAs; each CTA drains its own 128 accumulator rows.  No multicast anywhere.
//
// NH = 1: 256 x 256 tiles.  An SM pulls 32 KiB of operands per 64-k step (instead of the 48 KiB
// of the single-CTA kernel), the ring is 6 stages deep and the two 256-column accumulators in
// tensor memory alternate between consecutive tiles, so a tile's drain overlaps the next
// tile's main loop.
// NH = 2: 256 x 512 tiles, the two accumulators being the two 256-column halves of one tile.
// An SM then pulls 48 KiB per 64-k step for twice the flops: a quarter less L2 -> SM operand
// traffic per flop, which is what the tensor pipe waits for (and what the power cap bills).
// The drain still overlaps: half 0 of a tile is drained while the MMAs of half 1 of its last k
// step run, and the next tile's first MMAs into a half wait only for that half to be drained.
// 4 stages of 48 KiB.
constexpr int kPairStagesMax = 6;
constexpr int kPairBBytes = (BN / 2) * BK * 2;                 // 16 KiB: one CTA's share of a 256-column block

template <int NH>
struct PairCfg {
  static constexpr int kStages = NH == 1 ? 6 : 4;
  static constexpr int kStageBytes = kABytes + NH * kPairBBytes;   // 32 / 48 KiB per CTA
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

struct PairBarriers {
  uint64_t full[kPairStagesMax], empty[kPairStagesMax], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Accumulator slot and how many times it has been used before, for block `half` of the CTA
// pair's `local_tile`-th tile.
template <int NH>
__device__ __forceinline__ void acc_slot(uint32_t local_tile, uint32_t half, uint32_t& slot, uint32_t& use) {
  if (NH == 1) { slot = local_tile & 1; use = local_tile >> 1; }
  else { slot = half; use = local_tile; }
}

template <int NH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ GemmParams P) {
  using Cfg = PairCfg<NH>;
  constexpr int kPairStages = Cfg::kStages, kPairStageBytes = Cfg::kStageBytes;
  constexpr int BNT = BN * NH;     // tile width
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* gen_tiles = smem_raw + (tiles - raw);
  uint8_t* staging = gen_tiles + kPairStages * kPairStageBytes;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(staging + kStagingBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bars->acc_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[a]), 2 * kEpilogueWarps);   // the epilogue warps of both CTAs
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(&bars->tmem_base), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tiles_m = (P.M + 2 * BM - 1) / (2 * BM);
  const uint32_t num_tiles = tiles_m * P.tiles_n * P.batch * P.heads;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      TSB_PROF_DECL
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        uint32_t tm, tn, b, h;
        decode_tile(P, tile, tiles_m, tm, tn, b, h);
        const int bb = P.b_batched ? (int)b : 0;
        for (uint32_t kb = 0; kb < P.k_blocks; ++kb, ++it) {
          const uint32_t s = it % kPairStages, ph = (it / kPairStages) & 1;
#ifdef TSB_TUNING
          if (P.tune_noload & 2) { ok = false; break; }   // experiment: MMAs alone, no ring at all
#endif
          TSB_PROF_BEGIN
#ifdef TSB_TUNING
          if (P.tune_hint) {
            if (!ptx::mbar_wait_bounded_idle(ptx::smem_u32(&bars->empty[s]), ph ^ 1, abort_flag, kWaitLimit,
                                             (uint32_t)P.tune_hint)) { ok = false; break; }
          } else
#endif
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->empty[s]), ph ^ 1, abort_flag,
                                      kWaitLimit)) { ok = false; break; }
          TSB_PROF_END(prof_a)
          const uint32_t full_local = ptx::smem_u32(&bars->full[s]);
          const uint32_t full_leader = ptx::map_to_cta(full_local, 0);
#ifdef TSB_TUNING
          if ((P.tune_noload & 1) && it >= (uint32_t)kPairStages) {
            if (rank == 0) ptx::mbar_arrive(full_local);
            continue;
          }
#endif
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * kPairStageBytes);
          const uint32_t sa = tiles + s * kPairStageBytes, sb = sa + kABytes;
          ptx::tma_load_5d_pair(sa, &map_a, full_leader, 0, (int)(tm * 2 * BM + rank * BM), (int)b,
                                (int)kb, (int)h);
#pragma unroll
          for (int half = 0; half < NH; ++half) {
            const uint32_t sbh = sb + half * kPairBBytes;
            if (P.b_kmajor) {
              ptx::tma_load_5d_pair(sbh, &map_b, full_leader, 0,
                                    (int)(tn * BNT + half * BN + rank * (BN / 2)), bb, (int)kb, (int)h);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                ptx::tma_load_5d_pair(sbh + j * (BK * 128), &map_b, full_leader, 0, (int)(kb * BK), bb,
                                      (int)(tn * (BNT / 64) + half * (BN / 64) + rank * (BN / 128) + j),
                                      (int)h);
            }
          }
        }
      }
#ifdef TSB_TUNING
      if (rank == 0) {
        atomicAdd(&g_gemm_prof[3], (unsigned long long)prof_a);
        atomicAdd(&g_gemm_prof[4], (unsigned long long)(clock64() - prof_start));
      }
#endif
      // Let copies still in flight land before either CTA can exit.  On the normal path every
      // issued stage has been consumed by then and these waits return at once.  The "full"
      // barriers live in the leader and count both CTAs' bytes, so the leader waits on them
      // (ignoring the abort flag, which is what brought it here on the unwinding path); the
      // other CTA cannot observe them, so when it unwinds it simply lets a bounded time pass
      // that is far longer than a copy takes.  Both CTAs then meet in cluster_sync_all below.
      if (rank == 0) {
        const uint32_t issued = it < (uint32_t)kPairStages ? it : (uint32_t)kPairStages;
        for (uint32_t k = 0; k < issued; ++k) {
          const uint32_t j = it - 1 - k, s = j % kPairStages, ph = (j / kPairStages) & 1;
          ptx::mbar_wait_drain(ptx::smem_u32(&bars->full[s]), ph, kDrainLimit);
        }
      } else if (!ok) {
        ptx::spin_cycles(kDrainLimit);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      // (descriptor arithmetic as in the single-CTA kernel: constant high words, small adds)
      const uint32_t idesc = ptx::idesc_f16_f32(2 * BM, BN, 0, P.b_kmajor ? 0 : 1);
      const uint64_t da0 = ptx::smem_desc_sw128(tiles, 16, 1024);
      const uint64_t db0 = P.b_kmajor ? ptx::smem_desc_sw128(tiles + kABytes, 16, 1024)
                                      : ptx::smem_desc_sw128(tiles + kABytes, BK * 128, 1024);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t b_step = P.b_kmajor ? (32u >> 4) : (2048u >> 4);
      const uint32_t full0 = ptx::smem_u32(&bars->full[0]);
      const uint32_t empty_c0 = ptx::map_to_cta(ptx::smem_u32(&bars->empty[0]), 0);
      const uint32_t empty_c1 = ptx::map_to_cta(ptx::smem_u32(&bars->empty[0]), 1);
      uint32_t s = 0, ph = 0, local_tile = 0;
      bool ok = true;
      TSB_PROF_DECL
#ifdef TSB_TUNING
      unsigned long long prof_ns0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_ns0));
#endif
      for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++local_tile) {
        for (uint32_t kb = 0; ok && kb < P.k_blocks; ++kb) {
          TSB_PROF_BEGIN
#ifdef TSB_TUNING
          if (!(P.tune_noload & 2))
#endif
          if (!ptx::mbar_wait_bounded(full0 + s * 8, ph, abort_flag, kWaitLimit)) {
            ok = false;
            break;
          }
          TSB_PROF_END(prof_a)
#ifdef TSB_TUNING
          if (!(P.tune_noload & 4))
#endif
          ptx::tc_fence_after_sync();
          const uint32_t so = s * (kPairStageBytes >> 4);
          bool interleave = NH == 2 && kb != 0;
#ifdef TSB_TUNING
          if (P.tune_collect == 2) interleave = false;      // experiment: the plain order throughout
#endif
          if (interleave) {
            // Both halves of the tile use the same A k-slices.  From the second k block on (the first
            // still waits for the two accumulators one after the other, so that the left half can
            // start while the right one is being drained) the two MMAs of a k slice are issued back
            // to back, the first keeping A in the tensor core's collector buffer and the second
            // taking it from there: A is read from shared memory once instead of twice (a sixth of
            // the operand bytes of a k slice), which under the power cap is worth 3-5 %.
            uint32_t a_lo = (uint32_t)da0 + so, b_lo = (uint32_t)db0 + so;
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16) {
              const uint64_t ad = ((uint64_t)a_hi << 32) | a_lo;
              ptx::umma_f16_pair_a_fill(tmem_base, ad, ((uint64_t)b_hi << 32) | b_lo, idesc, 1u);
              ptx::umma_f16_pair_a_lastuse(tmem_base + BN, ad, ((uint64_t)b_hi << 32) | (b_lo + (kPairBBytes >> 4)),
                                           idesc, 1u);
              a_lo += 32u >> 4;
              b_lo += b_step;
            }
            if (kb + 1 == P.k_blocks) {   // the tile is complete once the MMAs issued so far are
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                const uint32_t f = ptx::smem_u32(&bars->acc_full[half]);
                ptx::umma_commit_pair(ptx::map_to_cta(f, 0));
                ptx::umma_commit_pair(ptx::map_to_cta(f, 1));
              }
            }
          } else
#pragma unroll
          for (int half = 0; half < NH; ++half) {
            uint32_t slot, use;
            acc_slot<NH>(local_tile, half, slot, use);
            if (kb == 0) {   // the block's accumulator must have been drained by both CTAs
              TSB_PROF_BEGIN
              if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->acc_empty[slot]), (use & 1) ^ 1, abort_flag,
                                          kWaitLimit)) { ok = false; break; }
              TSB_PROF_END(prof_b)
              ptx::tc_fence_after_sync();
            }
            const uint32_t d_tmem = tmem_base + slot * BN;
            uint32_t a_lo = (uint32_t)da0 + so, b_lo = (uint32_t)db0 + so + half * (kPairBBytes >> 4);
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16) {
              ptx::umma_f16_pair(d_tmem, ((uint64_t)a_hi << 32) | a_lo, ((uint64_t)b_hi << 32) | b_lo,
                                 idesc, k16 ? 1u : kb);
              a_lo += 32u >> 4;
              b_lo += b_step;
            }
            if (kb + 1 == P.k_blocks) {   // this block is complete once the MMAs issued so far are
              const uint32_t f = ptx::smem_u32(&bars->acc_full[slot]);
              ptx::umma_commit_pair(ptx::map_to_cta(f, 0));
              ptx::umma_commit_pair(ptx::map_to_cta(f, 1));
            }
          }
#ifdef TSB_TUNING
          if (!(P.tune_noload & 2)) {
#endif
          // (one masked commit for both CTAs instead of these two measured the same)
          ptx::umma_commit_pair(empty_c0 + s * 8);
          ptx::umma_commit_pair(empty_c1 + s * 8);
#ifdef TSB_TUNING
          }
#endif
          if (++s == kPairStages) { s = 0; ph ^= 1; }
        }
      }
#ifdef TSB_TUNING
      atomicAdd(&g_gemm_prof[0], (unsigned long long)prof_a);
      atomicAdd(&g_gemm_prof[1], (unsigned long long)prof_b);
      atomicAdd(&g_gemm_prof[2], (unsigned long long)(clock64() - prof_start));
      if (pair == 0) {   // SM cycles against wall-clock nanoseconds: the clock this launch really ran at
        unsigned long long ns1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns1));
        atomicAdd(&g_gemm_prof[5], (unsigned long long)(clock64() - prof_start));
        atomicAdd(&g_gemm_prof[6], ns1 - prof_ns0);
        atomicAdd(&g_gemm_prof[7], 1ull);
      }
#endif
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const uint32_t q = warp & 3;
    const uint32_t ch = (uint32_t)(warp - 2) >> 2;   // which 128 columns of a 256-column block
    uint8_t* my_stage = staging + (warp - 2) * (32 * 128);
    uint32_t local_tile = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < num_tiles; tile += num_pairs, ++local_tile) {
      uint32_t tm, tn, b, h;
      decode_tile(P, tile, tiles_m, tm, tn, b, h);
#pragma unroll 1
      for (int half = 0; half < NH; ++half) {
        uint32_t slot, use;
        acc_slot<NH>(local_tile, half, slot, use);
#ifdef TSB_TUNING
        if (P.tune_hint) {
          if (!ptx::mbar_wait_bounded_idle(ptx::smem_u32(&bars->acc_full[slot]), use & 1, abort_flag, kWaitLimit,
                                           (uint32_t)P.tune_hint)) { ok = false; break; }
        } else
#endif
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->acc_full[slot]), use & 1, abort_flag,
                                    kWaitLimit)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        auto release = [&] {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0)
            ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&bars->acc_empty[slot]), 0));
        };
        if (P.swiglu)
          drain_rows_swiglu(P, tmem_base + ((q * 32u) << 16) + slot * BN + ch * 128, my_stage,
                            tm * 2 * BM + rank * BM + q * 32, tn * BNT + half * BN + ch * 128, b, h, lane, release);
        else if (P.residual)
          drain_rows<true>(P, tmem_base + ((q * 32u) << 16) + slot * BN + ch * 128, my_stage,
                           tm * 2 * BM + rank * BM + q * 32, tn * BNT + half * BN + ch * 128, b, h, lane, release);
        else
          drain_rows<false>(P, tmem_base + ((q * 32u) << 16) + slot * BN + ch * 128, my_stage,
                            tm * 2 * BM + rank * BM + q * 32, tn * BNT + half * BN + ch * 128, b, h, lane, release);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other works
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(&g_gemm_error, 1);
}

// ---- host side --------------------------------------------------------------------

int g_sm_count = 0;

}  // namespace
}  // namespace tsb

using namespace tsb;

static int gemm_launch(const void* a, int64_t a_stick_stride, int64_t a_head_stride,
                       const void* b, int64_t b_stick_stride, int64_t b_head_stride,
                       const void* bias, const void* residual, void* c, int64_t c_stick_stride,
                       int64_t c_head_stride, int64_t heads, int64_t batch, int64_t M,
                       int64_t N, int64_t K, int b_kmajor, int b_batched, void* stream,
                       int swiglu = 0, void* const* c_owner = nullptr, int owners = 0, int owner_store = 0) {
  if ((uintptr_t)residual % 16) return TS_ERR_ALIGNMENT;
  if (owners) {
    if (owners < 1 || owners > 8 || !c_owner || residual || bias || swiglu || batch != 1 || heads != 1)
      return TS_ERR_INVALID;
    if (M % owners || (M / owners) % 32) return TS_ERR_UNSUPPORTED;
    for (int r = 0; r < owners; ++r)
      if (!c_owner[r] || (uintptr_t)c_owner[r] % 128) return TS_ERR_ALIGNMENT;
    c = c_owner[0];
  }
  if (swiglu && (N % 128 != 0 || bias || residual)) return TS_ERR_UNSUPPORTED;
  if (heads < 0 || batch < 0 || M < 0 || N < 0 || K < 0) return TS_ERR_INVALID;
  if (heads == 0 || batch == 0 || M == 0 || N == 0) return TS_OK;
  if (!a || !b || !c) return TS_ERR_INVALID;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)bias) % 128) return TS_ERR_ALIGNMENT;
  if (K == 0) return TS_ERR_UNSUPPORTED;
  if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31) || batch * heads >= (1ll << 31))
    return TS_ERR_TOO_LARGE;
  const int64_t ks = ceil_div(K, BK), ns = ceil_div(N, 64);
  const int64_t bb = b_batched ? batch : 1;
  // default strides: each operand is the whole stick image of its own [batch, rows, cols] tensor
  if (a_stick_stride <= 0) a_stick_stride = batch * M * kStickHalfs;
  if (b_stick_stride <= 0) b_stick_stride = bb * (b_kmajor ? N : K) * kStickHalfs;
  if (c_stick_stride <= 0) c_stick_stride = batch * M * kStickHalfs;
  if (heads > 1 && (a_head_stride <= 0 || b_head_stride < 0 || c_head_stride <= 0)) return TS_ERR_INVALID;
  if ((a_stick_stride | a_head_stride | b_stick_stride | b_head_stride | c_stick_stride | c_head_stride) % 8)
    return TS_ERR_ALIGNMENT;
  GemmParams P{};
  P.c = (__half*)c;
  P.bias = (const __half*)bias;
  P.residual = (const __half*)residual;
  P.swiglu = swiglu ? 1 : 0;
  P.M = (uint32_t)M; P.N = (uint32_t)N; P.K = (uint32_t)K;
  P.batch = (uint32_t)batch; P.heads = (uint32_t)heads;
  P.c_stick_stride = c_stick_stride;
  P.c_head_stride = c_head_stride;
  P.owners = (uint32_t)owners;
  P.owner_store = (uint32_t)owner_store;
  if (owners) {
    P.rows_per_owner = (uint32_t)(M / owners);
    P.c_stick_stride = (int64_t)P.rows_per_owner * kStickHalfs;   // every owner's buffer is the image of [M / owners, N]
    for (int r = 0; r < owners; ++r) P.c_owner[r] = (__half*)c_owner[r];
  }
  P.tiles_m = (uint32_t)ceil_div(M, BM);
  P.tiles_n = (uint32_t)ceil_div(N, BN);
  const int64_t tiles = (int64_t)P.tiles_m * P.tiles_n * batch * heads;
  if (tiles >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  P.num_tiles = (uint32_t)tiles;
  P.k_blocks = (uint32_t)ks;
  P.b_kmajor = b_kmajor ? 1 : 0;
  P.b_batched = b_batched ? 1 : 0;

  static std::once_flag once;
  std::call_once(once, [] {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  });
  // CTA pairs whenever a 256-row tile has work for both halves; 512-wide pair tiles when that
  // does not cost more in the last, partly filled wave than it saves in operand traffic.
  const int sms = g_sm_count > 0 ? g_sm_count : 148;
  bool use_pair = M > BM;
  int nh = 1;
  if (use_pair) {
    const int64_t pairs = sms / 2, tm2 = ceil_div(M, 2 * BM);
    const int64_t t1 = tm2 * ceil_div(N, BN) * batch * heads, t2 = tm2 * ceil_div(N, 2 * BN) * batch * heads;
    // time in units of one 256 x 256 tile: whole waves, a 512-wide tile costing kWideCost of two
    const double cost1 = (double)ceil_div(t1, pairs), cost2 = 2.0 * kWideCost * (double)ceil_div(t2, pairs);
    if (N > BN && cost2 < cost1) nh = 2;
  }
  uint32_t band = 8;
#ifdef TSB_TUNING
  // experiment hooks of the tuning build only (never compiled into the product library)
  if (const char* e = getenv("TS_GEMM_PAIR")) use_pair = atoi(e) != 0 && M > BM;
  if (const char* e = getenv("TS_GEMM_NH")) nh = atoi(e) == 2 && use_pair ? 2 : 1;
  if (const char* e = getenv("TS_GEMM_BAND")) band = (uint32_t)std::max(1, atoi(e));
  P.tune_noload = getenv("TS_GEMM_NOLOAD") ? atoi(getenv("TS_GEMM_NOLOAD")) : 0;
  P.tune_hint = getenv("TS_GEMM_HINT") ? atoi(getenv("TS_GEMM_HINT")) : 0;
  P.tune_epi = getenv("TS_GEMM_EPI") ? atoi(getenv("TS_GEMM_EPI")) : 0;
  P.tune_collect = getenv("TS_GEMM_COLLECT") ? atoi(getenv("TS_GEMM_COLLECT")) : 0;
#endif
  P.band_tiles = band;
  if (use_pair) P.tiles_n = (uint32_t)ceil_div(N, BN * nh);
  CUtensorMap map_a, map_b;
  if (!make_stick_map(&map_a, a, (uint64_t)M, (uint64_t)batch, (uint64_t)ks, (uint64_t)heads, a_stick_stride,
                a_head_stride, BM))
    return TS_ERR_CUDA;
  // a head stride of 0 shares one B between all heads
  const uint64_t b_heads = (heads > 1 && b_head_stride > 0) ? (uint64_t)heads : 1;
  const bool okb = b_kmajor ? make_stick_map(&map_b, b, (uint64_t)N, (uint64_t)bb, (uint64_t)ks, b_heads,
                                       b_stick_stride, b_head_stride, use_pair ? BN / 2 : BN)
                            : make_stick_map(&map_b, b, (uint64_t)K, (uint64_t)bb, (uint64_t)ns, b_heads,
                                       b_stick_stride, b_head_stride, BK);
  if (!okb) return TS_ERR_CUDA;
  if (b_heads == 1 && heads > 1) return TS_ERR_UNSUPPORTED;  // kernel indexes B by head

  static cudaError_t attr_err = cudaSuccess;
  if (use_pair) {
    const int64_t tiles2 = (int64_t)ceil_div(M, 2 * BM) * P.tiles_n * batch * heads;
    const int64_t pairs = std::min<int64_t>(tiles2, sms / 2);
    if (nh == 2) {
      attr_err = cudaFuncSetAttribute(gemm_f16_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PairCfg<2>::kSmemBytes);
      if (attr_err != cudaSuccess) { note_cuda_error(attr_err); return TS_ERR_CUDA; }
      gemm_f16_pair_kernel<2><<<(uint32_t)(2 * pairs), kThreads, PairCfg<2>::kSmemBytes, (cudaStream_t)stream>>>(
          map_a, map_b, P);
    } else {
      attr_err = cudaFuncSetAttribute(gemm_f16_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PairCfg<1>::kSmemBytes);
      if (attr_err != cudaSuccess) { note_cuda_error(attr_err); return TS_ERR_CUDA; }
      gemm_f16_pair_kernel<1><<<(uint32_t)(2 * pairs), kThreads, PairCfg<1>::kSmemBytes, (cudaStream_t)stream>>>(
          map_a, map_b, P);
    }
    TSB_CHECK_LAUNCH();
    return TS_OK;
  }
  attr_err = cudaFuncSetAttribute(gemm_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBytes);  // per device, idempotent
  if (attr_err != cudaSuccess) { note_cuda_error(attr_err); return TS_ERR_CUDA; }
  const uint32_t grid = (uint32_t)std::min<int64_t>(tiles, g_sm_count > 0 ? g_sm_count : 148);
  gemm_f16_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(map_a, map_b, P);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

extern "C" int ts_gemm_f16_ex(const void* a, int64_t a_stick_stride, int64_t a_head_stride,
                              const void* b, int64_t b_stick_stride, int64_t b_head_stride,
                              const void* bias, void* c, int64_t c_stick_stride,
                              int64_t c_head_stride, int64_t heads, int64_t batch, int64_t M,
                              int64_t N, int64_t K, int b_kmajor, int b_batched, void* stream) {
  return gemm_launch(a, a_stick_stride, a_head_stride, b, b_stick_stride, b_head_stride, bias, nullptr,
                     c, c_stick_stride, c_head_stride, heads, batch, M, N, K, b_kmajor, b_batched,
                     stream);
}

extern "C" int ts_gemm_f16(const void* a, const void* b, const void* bias, void* c, int64_t batch,
                           int64_t M, int64_t N, int64_t K, int b_kmajor, int b_batched,
                           void* stream) {
  return gemm_launch(a, 0, 0, b, 0, 0, bias, nullptr, c, 0, 0, 1, batch, M, N, K, b_kmajor, b_batched,
                     stream);
}

extern "C" int ts_gemm_f16_residual(const void* a, const void* b, const void* bias,
                                    const void* residual, void* c, int64_t batch, int64_t M,
                                    int64_t N, int64_t K, int b_kmajor, int b_batched, void* stream) {
  return gemm_launch(a, 0, 0, b, 0, 0, bias, residual, c, 0, 0, 1, batch, M, N, K, b_kmajor,
                     b_batched, stream);
}

// Synchronises the device and reports (and clears) the sticky error word the GEMM
// kernel sets when one of its bounded waits gave up.  Returns 0, 1 or an error code.
extern "C" int ts_gemm_error_state(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  }
  return v;
}

namespace tsb {
namespace {
// One warp waits, with the given limit, on a barrier nothing will ever arrive on: the unwinding
// path of the GEMM's bounded waits in isolation (no TMA copy, no MMA, no tensor memory involved).
__global__ void gemm_wait_selftest_kernel(long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  volatile int* flag = &abort_flag;
  const bool done = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, flag, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && (!done || abort_flag)) atomicExch(&g_gemm_error, 1);
}
}  // namespace
}  // namespace tsb

// Diagnostic: exercises the give-up path of the kernels' bounded waits.  A single warp waits
// `limit_cycles` SM clocks (clamped to [1000, 10^7]) for an arrival that never comes, then raises
// the same sticky error word a real kernel would: ts_gemm_error_state() reports 1 afterwards (and
// clears it).  Nothing else is in flight in that launch, so the device stays fully usable.
extern "C" int ts_gemm_wait_selftest(int64_t limit_cycles, void* stream) {
  const long long limit = limit_cycles < 1000 ? 1000 : (limit_cycles > 10000000 ? 10000000 : limit_cycles);
  gemm_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

extern "C" int ts_gemm_f16_scatter_add(const void* a, const void* b, void* const* c_owner, int owners,
                                       int64_t M, int64_t N, int64_t K, int b_kmajor, void* stream) {
  return gemm_launch(a, 0, 0, b, 0, 0, nullptr, nullptr, nullptr, 0, 0, 1, 1, M, N, K, b_kmajor, 0, stream, 0,
                     c_owner, owners);
}

extern "C" int ts_gemm_f16_scatter_store(const void* a, const void* b, void* const* c_owner, int owners,
                                         int64_t M, int64_t N, int64_t K, int b_kmajor, void* stream) {
  return gemm_launch(a, 0, 0, b, 0, 0, nullptr, nullptr, nullptr, 0, 0, 1, 1, M, N, K, b_kmajor, 0, stream, 0,
                     c_owner, owners, 1);
}

extern "C" int ts_gemm_f16_swiglu(const void* a, const void* w_gate_up, void* c, int64_t batch,
                                  int64_t M, int64_t N_out, int64_t K, void* stream) {
  if (N_out < 0) return TS_ERR_INVALID;
  if (N_out % 64 != 0) return TS_ERR_UNSUPPORTED;
  // the product has 2 * N_out columns; the result image has N_out: its default stick stride is
  // that of a dense [batch, M, N_out] image, which is also what the product's would be
  return gemm_launch(a, 0, 0, w_gate_up, 0, 0, nullptr, nullptr, c, 0, 0, 1, batch, M, 2 * N_out, K, 1, 0,
                     stream, 1);
}

#ifdef TSB_TUNING
// tuning build only: reads and clears the experiment counters
extern "C" int ts_gemm_prof(unsigned long long* out8) {
  if (cudaMemcpyFromSymbol(out8, g_gemm_prof, sizeof(unsigned long long) * 8) != cudaSuccess) return TS_ERR_CUDA;
  unsigned long long zero[8] = {0};
  cudaMemcpyToSymbol(g_gemm_prof, zero, sizeof(zero));
  return TS_OK;
}
#endif
