// Causal scaled-dot-product attention as one kernel on the 5th-generation tensor cores:
// the score matrix never leaves the SM (tensor memory -> registers -> shared memory).
//
// Operands are the packed stick images the projection GEMMs write, [batch*seq, heads*128]:
// head h owns stick columns 2h and 2h+1, so a 128-row x 128-wide tile of Q, K or V is two
// 128-row x 128-byte boxes, which TMA drops into shared memory in exactly the swizzled form
// tcgen05.mma reads (Q, K: K-major; V: MN-major).  The reference has no attention kernel
// (its decoder-layer test, tests/test_modules.py:178-211, is skipped); this stands in for the
// bmm / where / _softmax / bmm sequence its compiled path would emit.
//
// Two kernels, both with the probabilities kept in tensor memory (written over the scores they
// were computed from; the P V product takes its A operand from there):
//   * attention_causal_pair64_kernel, sequences of an even number of 128-row tiles: two query
//     tiles of one (batch, head) per CTA, 64-key steps, per tile two score buffers and the output;
//   * attention_causal_tmem_kernel, any other sequence: one query tile per CTA, 128-key steps, three
//     score buffers and the output.
// In both, one thread per tile issues the MMAs, producer lanes of warp 0 issue TMA (Q and K on one
// lane, V on another), and one softmax thread per query row runs the online softmax:
//     S_j = Q K_j^T,   P_j = exp2((S_j - m) c) -> fp16 over S_j,   l += rowsum P_j,   O += P_j V_j
// and at the end out = O / l.  m is the row maximum used as the exponent offset; it is only
// raised (and O, l rescaled, by the softmax threads through tcgen05.ld/st) when a row's new
// maximum exceeds it by more than 8 in the exponent, i.e. P stays <= 256, so in steady state
// the softmax threads never touch O.  Every wait is bounded; on a timeout the CTA raises a flag,
// every role leaves its loops, the producers wait (bounded) for their copies in flight, tensor
// memory is released and a sticky error word is set.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tma_map.cuh"

namespace tsb {
namespace {

constexpr int kTile = 128;                      // queries per tile = keys per tile = head dim
constexpr int kBlockBytes = kTile * 128;        // one 128-row x 64-lane box: 16 KiB
constexpr int kTileBytes = 2 * kBlockBytes;     // 32 KiB
constexpr uint32_t kAttnTmemCols = 512;         // every kernel here uses all of tensor memory
constexpr float kRescaleThreshold = 8.f;        // in units of the exponent (log2)
constexpr long long kAttnWaitLimit = 4000000000ll;  // ~2 s of SM clocks
constexpr long long kAttnDrainLimit = 200000ll;   // ~0.1 ms: far longer than a TMA copy is in flight

__device__ int g_attn_error;  // sticky: set when a bounded wait gave up
#ifdef TSB_TUNING
// experiment counters of the tuning build (two-tile kernel): cycles group A's MMA thread waited for
// K [0], for S to be taken [1], for V [2], for P [3], its loop [4]; cycles the first softmax warp of
// group A waited for S [5], for the previous P V [6], its loop [7]
__device__ unsigned long long g_attn_prof[8];
#define ATTN_PROF(idx, stmt) { const long long t0__ = clock64(); stmt; prof[idx] += clock64() - t0__; }
#else
#define ATTN_PROF(idx, stmt) { stmt; }
#endif

struct AttnParams {
  __half* out;
  uint32_t batch, seq, heads, q_tiles, num_items;
  int64_t stick_stride;   // elements between stick columns of the packed images
  float scale_log2;       // softmax scale * log2(e)
  uint32_t heads_per_round;   // two-tile kernel: (batch, head) slices in flight together; 0 = linear order
#ifdef TSB_TUNING
  int tune_mode;              // experiment: 1 = MMAs without the softmax (its warps leave at once)
#endif
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- two query tiles per CTA -----------------------------------------------------------
// For sequences of an even number of tiles.  A CTA takes the query tiles 2p ("A") and 2p+1 ("B")
// of one (batch, head) together: they share every K / V tile, and each has its own group of
// four softmax warps (one thread per query row), its own score buffers and output accumulator.
// While one group is in its exponentials the other one's waits and the MMAs of both run
// underneath.  Each group has its own MMA-issuing thread (warps 1 and 10), so that neither waits
// on the other's softmax; K and V are loaded by two different threads of the TMA warp, each
// waiting only for its own buffers (one thread loading K and V in turn would hold every K load
// back behind the V buffer).
constexpr int kPairAttnThreads = 352;   // TMA warp, MMA warp A, 8 softmax warps, MMA warp B

// Work order of the two-tile kernel.  The grid is heads_per_round x (pairs per head) CTAs; in
// round r CTA c works on (batch, head) slice r * heads_per_round + c / pairs and on tile pair
// number (c % pairs + r) % pairs of the sequence light, heavy, light, heavy, ... of it.  So the CTAs running together read the K / V of only
// heads_per_round slices (they stay in L2 for all the pairs of a slice), and over the rounds
// every CTA gets each pair index, light and heavy, equally often.  heads_per_round == 0 (more
// pairs per head than SMs): plain order, heaviest pairs first.
// When the slices left over after the last full round are no more than the SMs left over
// after heads_per_round * pairs, those spare CTAs take one left-over slice each, all its pairs,
// instead of a short last round that would land on CTAs already carrying a full share.
__device__ __forceinline__ void unit_layout(const AttnParams& P, uint32_t units, uint32_t& main_ctas,
                                            uint32_t& main_rounds, bool& spares_take_rest) {
  const uint32_t bh_count = P.batch * P.heads;
  main_ctas = P.heads_per_round * units;
  const uint32_t full = bh_count / P.heads_per_round, rest = bh_count % P.heads_per_round;
  // (a spare CTA then does a whole slice, `units` items, while the others do `full` items each: only
  // worth it when that is no more than their share)
  spares_take_rest = rest != 0 && rest <= gridDim.x - main_ctas && units <= full;
  main_rounds = full + ((rest != 0 && !spares_take_rest) ? 1 : 0);
}
// `units` = work items per (batch, head) slice: tile pairs for the two-tile kernels, tiles for the
// one-tile kernel.
__device__ __forceinline__ uint32_t unit_item_count(const AttnParams& P, uint32_t units) {
  const uint32_t bh_count = P.batch * P.heads;
  if (P.heads_per_round == 0) return units * bh_count;
  uint32_t main_ctas, main_rounds;
  bool spares;
  unit_layout(P, units, main_ctas, main_rounds, spares);
  return (main_rounds > units ? main_rounds : units) * gridDim.x;
}
__device__ __forceinline__ bool decode_unit_item(const AttnParams& P, uint32_t units, uint32_t item, uint32_t& pr,
                                                 uint32_t& b, uint32_t& h) {
  const uint32_t bh_count = P.batch * P.heads;
  uint32_t bh;
  if (P.heads_per_round == 0) {
    pr = units - 1 - item / bh_count;
    bh = item % bh_count;
  } else {
    uint32_t main_ctas, main_rounds;
    bool spares;
    unit_layout(P, units, main_ctas, main_rounds, spares);
    const uint32_t r = item / gridDim.x, c = item - r * gridDim.x;
    if (c < main_ctas) {
      if (r >= main_rounds) return false;
      bh = r * P.heads_per_round + c / units;
      const uint32_t k = (c % units + r) % units;
      pr = (k & 1) ? units - 1 - (k >> 1) : (k >> 1);   // 0, last, 1, last-1, ...: neighbours sum to a constant
    } else {
      if (!spares || r >= units) return false;
      bh = (bh_count / P.heads_per_round) * P.heads_per_round + (c - main_ctas);
      pr = units - 1 - r;                                // a whole slice, heaviest unit first
    }
    if (bh >= bh_count) return false;
  }
  b = bh % P.batch;
  h = bh / P.batch;
  return true;
}
__device__ __forceinline__ uint32_t pair_item_count(const AttnParams& P) { return unit_item_count(P, P.q_tiles / 2); }
__device__ __forceinline__ bool decode_pair_item(const AttnParams& P, uint32_t item, uint32_t& pr,
                                                 uint32_t& b, uint32_t& h) {
  return decode_unit_item(P, P.q_tiles / 2, item, pr, b, h);
}

// ---- two query tiles per CTA, 64 keys at a time, probabilities in tensor memory ----------------
// Keeping P in shared memory makes shared-memory bandwidth the limit (per 128-key step the tensor
// cores read 256 KiB of operands, the softmax threads store 64 KiB of P and TMA fills 64 KiB: 3000
// cycles' worth at 128 B per clock for 2048 cycles of MMAs; that form measured 0.41 ms at the
// benchmark shape and is no longer in the tree).  Here P never touches shared memory: the softmax threads write it (fp16, two per 32-bit column) over the
// scores they have just read, and the P V product takes its A operand from tensor memory.  So that
// scores can still be computed ahead of the softmax, a step is 64 keys: per group two 64-column
// score buffers (S(u+1) is computed while the softmax works on S(u)) plus the 128-column output,
// 256 columns, 512 for the two groups.
//   tensor memory: group A: S0 S1 O | group B: S0 S1 O   (64 + 64 + 128 columns each)
//   shared memory: Q_A Q_B | K (3 tiles of 128 keys) | V (2 tiles)
// A score buffer is free again once the P V product that read P from it has finished, so S(u+2)
// waits for P V(u).  K and V tiles are loaded whole (128 keys) by the two producer lanes and
// consumed in halves.
constexpr int kHalfKeys = 64;
constexpr int kP64KStages = 3, kP64VStages = 2;
constexpr int kP64SmemTiles = 2 + kP64KStages + kP64VStages;
constexpr int kP64Smem = kP64SmemTiles * kTileBytes + 1024 /*align*/ + 512 /*barriers*/;

struct P64Bars {
  uint64_t q_full, q_empty, k_full[kP64KStages], k_empty[kP64KStages], v_full[kP64VStages], v_empty[kP64VStages];
  uint64_t s_full[2][2], p_full[2][2], pv_done[2][2];   // [group][score buffer]
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(P64Bars) <= 512, "barrier block outgrew its shared-memory reservation");

__global__ void __launch_bounds__(kPairAttnThreads, 1)
attention_causal_pair64_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttnParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t sq = base, sk = sq + 2 * kTileBytes, sv = sk + kP64KStages * kTileBytes;
  P64Bars* bars = reinterpret_cast<P64Bars*>(gen_base + kP64SmemTiles * kTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;
  const uint32_t num_items = pair_item_count(P);

  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bars->q_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->q_empty), 2);        // released by both MMA threads
    for (int i = 0; i < kP64KStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->k_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->k_empty[i]), 2);
    }
    for (int i = 0; i < kP64VStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->v_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->v_empty[i]), 2);
    }
    for (int x = 0; x < 2; ++x)
      for (int b = 0; b < 2; ++b) {
        ptx::mbar_init(ptx::smem_u32(&bars->s_full[x][b]), 1);
        ptx::mbar_init(ptx::smem_u32(&bars->p_full[x][b]), 4);   // one arrival per softmax warp of the group
        ptx::mbar_init(ptx::smem_u32(&bars->pv_done[x][b]), 1);
      }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kAttnTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producers: lane 0 Q and K, lane 1 V
    if (lane == 0) {
      uint32_t kt = 0, item_n = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x, ++item_n) {
        uint32_t pr, b, h;
        if (!decode_pair_item(P, item, pr, b, h)) continue;
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->q_empty), (item_n & 1) ^ 1, abort_flag, kAttnWaitLimit)) break;
        const uint32_t qf = ptx::smem_u32(&bars->q_full);
        ptx::mbar_arrive_expect_tx(qf, 2 * kTileBytes);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int qrow = (int)((2 * pr + x) * kTile);
          ptx::tma_load_5d(sq + x * kTileBytes, &map_q, qf, 0, qrow, (int)b, (int)(2 * h), 0);
          ptx::tma_load_5d(sq + x * kTileBytes + kBlockBytes, &map_q, qf, 0, qrow, (int)b, (int)(2 * h + 1), 0);
        }
        const uint32_t n = 2 * pr + 2;
        for (uint32_t j = 0; j < n; ++j, ++kt) {
          const uint32_t st = kt % kP64KStages, ph = (kt / kP64KStages) & 1;
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->k_empty[st]), ph ^ 1, abort_flag, kAttnWaitLimit)) {
            ok = false;
            break;
          }
          const uint32_t kf = ptx::smem_u32(&bars->k_full[st]);
          ptx::mbar_arrive_expect_tx(kf, kTileBytes);
          ptx::tma_load_5d(sk + st * kTileBytes, &map_k, kf, 0, (int)(j * kTile), (int)b, (int)(2 * h), 0);
          ptx::tma_load_5d(sk + st * kTileBytes + kBlockBytes, &map_k, kf, 0, (int)(j * kTile), (int)b, (int)(2 * h + 1), 0);
        }
      }
      if (*abort_flag) {   // after an abort only: let copies in flight land before the CTA exits
        for (uint32_t k = 0; k < (kt < (uint32_t)kP64KStages ? kt : (uint32_t)kP64KStages); ++k) {
          const uint32_t t = kt - 1 - k;
          ptx::mbar_wait_drain(ptx::smem_u32(&bars->k_full[t % kP64KStages]), (t / kP64KStages) & 1, kAttnDrainLimit);
        }
        if (item_n > 0) ptx::mbar_wait_drain(ptx::smem_u32(&bars->q_full), (item_n - 1) & 1, kAttnDrainLimit);
      }
    } else if (lane == 1) {
      uint32_t kt = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        uint32_t pr, b, h;
        if (!decode_pair_item(P, item, pr, b, h)) continue;
        const uint32_t n = 2 * pr + 2;
        for (uint32_t j = 0; j < n; ++j, ++kt) {
          const uint32_t st = kt % kP64VStages, ph = (kt / kP64VStages) & 1;
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->v_empty[st]), ph ^ 1, abort_flag, kAttnWaitLimit)) {
            ok = false;
            break;
          }
          const uint32_t vf = ptx::smem_u32(&bars->v_full[st]);
          ptx::mbar_arrive_expect_tx(vf, kTileBytes);
          ptx::tma_load_5d(sv + st * kTileBytes, &map_v, vf, 0, (int)(j * kTile), (int)b, (int)(2 * h), 0);
          ptx::tma_load_5d(sv + st * kTileBytes + kBlockBytes, &map_v, vf, 0, (int)(j * kTile), (int)b, (int)(2 * h + 1), 0);
        }
      }
      if (*abort_flag)
        for (uint32_t k = 0; k < (kt < (uint32_t)kP64VStages ? kt : (uint32_t)kP64VStages); ++k) {
          const uint32_t t = kt - 1 - k;
          ptx::mbar_wait_drain(ptx::smem_u32(&bars->v_full[t % kP64VStages]), (t / kP64VStages) & 1, kAttnDrainLimit);
        }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------ MMA issuers: warp 1 for group A, warp 10 for B
    if (lane == 0) {
      const int x = warp == 1 ? 0 : 1;
      const uint32_t idesc_s = ptx::idesc_f16_f32(kTile, kHalfKeys, 0, 0);     // 128 queries x 64 keys
      const uint32_t idesc_pv = ptx::idesc_f16_f32(kTile, kTile, 0, 1);       // 128 queries x 128 dims, V MN-major
      const uint32_t qb = sq + x * kTileBytes;
      const uint32_t tg = tmem_base + x * 256;    // this group's columns: S0 S1 O
      uint32_t kt = 0, item_n = 0;   // key tiles of finished items; items done
      uint32_t U = 0;                // half-steps (64 keys) of finished items: phases of the per-buffer barriers
      auto ready = [&](uint64_t* bar, uint32_t parity) { return ptx::mbar_test_wait(ptx::smem_u32(bar), parity); };
      bool ok = true;
      for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x, ++item_n) {
        uint32_t pr, b, h;
        if (!decode_pair_item(P, item, pr, b, h)) continue;
        const uint32_t n = 2 * pr + 2;          // key tiles loaded for the item
        const uint32_t nx = n - 1 + x;          // key tiles this group uses (A stops one short)
        const uint32_t hx = 2 * nx, hn = 2 * n; // in half-steps
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->q_full), item_n & 1, abort_flag, kAttnWaitLimit)) break;
        uint32_t s_next = 0, p_next = 0;        // next half-step whose scores / whose P V product is to be issued
        const long long t_item = clock64();
        while (ok && p_next < hn) {
          bool progress = false;
          // scores of half-step s_next: at most two ahead of the P V products (two score buffers)
          if (s_next < hn && s_next < p_next + 2) {
            const uint32_t t = kt + (s_next >> 1), ks = t % kP64KStages, hf = s_next & 1, ug = U + s_next;
            bool can = ready(&bars->k_full[ks], (t / kP64KStages) & 1);
            if (can && s_next < hx && ug >= 2)   // the buffer's previous P has been consumed
              can = ready(&bars->pv_done[x][ug & 1], ((ug - 2) >> 1) & 1);
            if (can) {
              if (s_next < hx) {
                ptx::tc_fence_after_sync();
                const uint32_t kb = sk + ks * kTileBytes + hf * (kHalfKeys * 128);
#pragma unroll
                for (int k16 = 0; k16 < kTile / 16; ++k16) {
                  const uint32_t off = (k16 >> 2) * kBlockBytes + (k16 & 3) * 32;
                  ptx::umma_f16(tg + (ug & 1) * kHalfKeys, ptx::smem_desc_sw128(qb + off, 16, 1024),
                                ptx::smem_desc_sw128(kb + off, 16, 1024), idesc_s, k16 != 0);
                }
                ptx::umma_commit(ptx::smem_u32(&bars->s_full[x][ug & 1]));
                if (s_next + 1 == hx) ptx::umma_commit(ptx::smem_u32(&bars->q_empty));   // Q_x is not read again
              }
              if (hf == 1) ptx::umma_commit(ptx::smem_u32(&bars->k_empty[ks]));   // both halves of the K tile are done with
              ++s_next;
              progress = true;
            }
          }
          // P V product of half-step p_next
          if (p_next < s_next) {
            const uint32_t t = kt + (p_next >> 1), vs = t % kP64VStages, hf = p_next & 1, ug = U + p_next;
            bool can = ready(&bars->v_full[vs], (t / kP64VStages) & 1);
            if (can && p_next < hx) can = ready(&bars->p_full[x][ug & 1], (ug >> 1) & 1);
#ifdef TSB_TUNING
            if (P.tune_mode == 1) can = ready(&bars->v_full[vs], (t / kP64VStages) & 1);
#endif
            if (can) {
              if (p_next < hx) {
                ptx::tc_fence_after_sync();
                const uint32_t vb = sv + vs * kTileBytes;
#pragma unroll
                for (int kk = 0; kk < kHalfKeys / 16; ++kk) {
                  const uint64_t db = ptx::smem_desc_sw128(vb + (hf * 4 + kk) * 2048, kBlockBytes, 1024);
                  ptx::umma_f16_ts(tg + 128, tg + (ug & 1) * kHalfKeys + kk * 8, db, idesc_pv,
                                   (p_next ? 1u : 0u) | (uint32_t)kk);
                }
                ptx::umma_commit(ptx::smem_u32(&bars->pv_done[x][ug & 1]));
              }
              if (hf == 1) ptx::umma_commit(ptx::smem_u32(&bars->v_empty[vs]));
              ++p_next;
              progress = true;
            }
          }
          if (!progress) {
            if (*abort_flag) { ok = false; break; }
            if (clock64() - t_item > kAttnWaitLimit) { *abort_flag = 1; ok = false; break; }
          }
        }
        kt += n;
        U += hx;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax + output: group A = warps 2-5, B = 6-9
    const uint32_t x = (uint32_t)(warp - 2) >> 2;
    const uint32_t quarter = warp & 3;              // TMEM lane quarter this warp may read
    const uint32_t row = quarter * 32 + lane;
    const uint32_t tg = tmem_base + ((quarter * 32u) << 16) + x * 256, to = tg + 128;
    const float c = P.scale_log2;
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(bar), parity, abort_flag,
                                                            kAttnWaitLimit)) != 0;
    };
    uint32_t U = 0;   // half-steps this group has processed in earlier items
    bool ok = true;
#ifdef TSB_TUNING
    if (P.tune_mode == 1) ok = false;
#endif
    for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      uint32_t pr, b, h;
      if (!decode_pair_item(P, item, pr, b, h)) continue;
      const uint32_t qt = 2 * pr + x, hx = 2 * (qt + 1);
      float m = -1e30f, l = 0.f;
      for (uint32_t u = 0; u < hx; ++u) {
        const uint32_t ug = U + u, buf = ug & 1, ts = tg + buf * kHalfKeys;
        if (!warp_wait(&bars->s_full[x][buf], (ug >> 1) & 1)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        uint32_t r[2][32];
        ptx::tmem_ld_32x32(ts, r[0]);
        ptx::tmem_ld_32x32(ts + 32, r[1]);
        ptx::tmem_ld_wait();
        if ((u >> 1) == qt) {   // diagonal tile: keys after the query do not exist
          const uint32_t key0 = (u & 1) * kHalfKeys;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (key0 + (uint32_t)(ch * 32 + i) > row) r[ch][i] = 0xff800000u;   // -inf
        }
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(r[ch][i]));
        const float tile_max = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                     fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        if (u == 0) {
          m = tile_max;   // key 0 exists for every query, so this is finite
        } else if (__any_sync(0xffffffffu, (tile_max - m) * c > kRescaleThreshold)) {
          // raise the exponent offset (lazily): O and l shrink by alpha.  O must be at rest: the latest
          // P V product of this group is the one of the previous half-step.
          if (!warp_wait(&bars->pv_done[x][(ug - 1) & 1], ((ug - 1) >> 1) & 1)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const float m_new = fmaxf(m, tile_max);
          const float alpha = ex2f((m - m_new) * c);
          l *= alpha;
          m = m_new;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            ptx::tmem_ld_32x32(to + ch * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ptx::tmem_st_32x32(to + ch * 32, o);
          }
          ptx::tmem_st_wait();
        }
        const float mc = m * c;
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t packed[32];
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2f(fmaf(__uint_as_float(r[ch][i]), c, -mc));
            const float p1 = ex2f(fmaf(__uint_as_float(r[ch][i + 1]), c, -mc));
            sum[(i >> 1) & 3] += p0 + p1;
            const __half2 hp = __floats2half2_rn(p0, p1);
            packed[ch * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&hp);
          }
        l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
        ptx::tmem_st_32x32(ts, packed);   // P over the scores just read: keys 2c, 2c+1 in column c
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->p_full[x][buf]));
      }
      if (!ok) break;
      U += hx;
      // both score buffers' last P V products (hx is even and at least 2)
      if (!warp_wait(&bars->pv_done[x][0], ((U - 2) >> 1) & 1) || !warp_wait(&bars->pv_done[x][1], ((U - 1) >> 1) & 1)) break;
      ptx::tc_fence_after_sync();
      const float inv = 1.f / l;
      const bool row_ok = qt * kTile + row < P.seq;
      const int64_t grow = (int64_t)b * P.seq + (int64_t)qt * kTile + row;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        ptx::tmem_ld_32x32(to + ch * 32, o);
        ptx::tmem_ld_wait();
        __half* dst = P.out + (int64_t)(2 * h + (ch >> 1)) * P.stick_stride + grow * kStickHalfs + (ch & 1) * 32;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          Vec8h ov;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = v * 8 + 2 * e;
            ov.h2[e] = __floats2half2_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
          }
          if (row_ok) st_global_v4(dst + v * 8, ov.u);
        }
      }
      ptx::tc_fence_before_sync();
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kAttnTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(&g_attn_error, 1);
}

// ---- one query tile per CTA, 128 keys at a time, probabilities in tensor memory -----------------
// The two-tile kernel above is held back by its 64-key score MMAs (a 128x64x16 MMA occupies the
// tensor pipe as long as a 128x128x16 one).  With one query tile per CTA the 512 columns hold three
// full-width score buffers and the output:
//   tensor memory: S0 S1 S2 O   (128 columns each)      shared memory: Q | K (3 tiles) | V (3 tiles)
// so the scores run two key tiles ahead of the softmax threads: the buffer that S(j+2) goes into
// was last read by P V(j-1), which finished a step ago, so the chain P(j) -> P V(j) -> "done" ->
// next scores never delays the softmax (with two buffers it did: S(j+2) had to wait for P V(j)).
// Every MMA is 128 wide.  One softmax thread per query row (four warps, the row's 128 scores in
// registers); P goes back over the scores it was computed from and the P V product reads it from
// there.  (Measured and dropped: two threads per row sharing its columns, and two sets of warps
// taking alternate steps; both lose more to the 168-register limit of a 10-warp CTA and to the
// hand-offs than the overlap gains.)  CTAs that run together share the K / V of a few
// (batch, head) slices through the work order of decode_unit_item.
constexpr int kT1Threads = 192;                  // producer warp, MMA warp, 4 softmax warps
constexpr int kT1KStages = 3, kT1VStages = 3;
constexpr int kT1SmemTiles = 1 + kT1KStages + kT1VStages;

struct T1Bars {
  uint64_t q_full, q_empty, k_full[kT1KStages], k_empty[kT1KStages], v_full[kT1VStages], v_empty[kT1VStages];
  uint64_t s_full[3], p_full[3], pv_done[3];   // per score buffer
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(T1Bars) <= 512, "barrier block outgrew its shared-memory reservation");
constexpr int kT1Smem = kT1SmemTiles * kTileBytes + 1024 /*align*/ + 512 /*barriers*/;

__global__ void __launch_bounds__(kT1Threads, 1)
attention_causal_tmem_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttnParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t sq = base, sk = sq + kTileBytes, sv = sk + kT1KStages * kTileBytes;
  T1Bars* bars = reinterpret_cast<T1Bars*>(gen_base + kT1SmemTiles * kTileBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;
  const uint32_t units = P.q_tiles;
  const uint32_t num_items = unit_item_count(P, units);

  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bars->q_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->q_empty), 1);
    for (int i = 0; i < kT1KStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->k_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->k_empty[i]), 1);
    }
    for (int i = 0; i < kT1VStages; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bars->v_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->v_empty[i]), 1);
    }
    for (int b = 0; b < 3; ++b) {
      ptx::mbar_init(ptx::smem_u32(&bars->s_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[b]), 4);   // one arrival per softmax warp
      ptx::mbar_init(ptx::smem_u32(&bars->pv_done[b]), 1);
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), kAttnTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producers: lane 0 Q and K, lane 1 V
    if (lane == 0) {
      uint32_t kt = 0, item_n = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        uint32_t qt, b, h;
        if (!decode_unit_item(P, units, item, qt, b, h)) continue;
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->q_empty), (item_n & 1) ^ 1, abort_flag, kAttnWaitLimit)) break;
        ++item_n;
        const uint32_t qf = ptx::smem_u32(&bars->q_full);
        ptx::mbar_arrive_expect_tx(qf, kTileBytes);
        ptx::tma_load_5d(sq, &map_q, qf, 0, (int)(qt * kTile), (int)b, (int)(2 * h), 0);
        ptx::tma_load_5d(sq + kBlockBytes, &map_q, qf, 0, (int)(qt * kTile), (int)b, (int)(2 * h + 1), 0);
        for (uint32_t j = 0; j <= qt; ++j, ++kt) {
          const uint32_t st = kt % kT1KStages, ph = (kt / kT1KStages) & 1;
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->k_empty[st]), ph ^ 1, abort_flag, kAttnWaitLimit)) {
            ok = false;
            break;
          }
          const uint32_t kf = ptx::smem_u32(&bars->k_full[st]);
          ptx::mbar_arrive_expect_tx(kf, kTileBytes);
          ptx::tma_load_5d(sk + st * kTileBytes, &map_k, kf, 0, (int)(j * kTile), (int)b, (int)(2 * h), 0);
          ptx::tma_load_5d(sk + st * kTileBytes + kBlockBytes, &map_k, kf, 0, (int)(j * kTile), (int)b, (int)(2 * h + 1), 0);
        }
      }
      if (*abort_flag) {   // after an abort only: let copies in flight land before the CTA exits
        for (uint32_t k = 0; k < (kt < (uint32_t)kT1KStages ? kt : (uint32_t)kT1KStages); ++k) {
          const uint32_t t = kt - 1 - k;
          ptx::mbar_wait_drain(ptx::smem_u32(&bars->k_full[t % kT1KStages]), (t / kT1KStages) & 1, kAttnDrainLimit);
        }
        if (item_n > 0) ptx::mbar_wait_drain(ptx::smem_u32(&bars->q_full), (item_n - 1) & 1, kAttnDrainLimit);
      }
    } else if (lane == 1) {
      uint32_t kt = 0;
      bool ok = true;
      for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        uint32_t qt, b, h;
        if (!decode_unit_item(P, units, item, qt, b, h)) continue;
        for (uint32_t j = 0; j <= qt; ++j, ++kt) {
          const uint32_t st = kt % kT1VStages, ph = (kt / kT1VStages) & 1;
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bars->v_empty[st]), ph ^ 1, abort_flag, kAttnWaitLimit)) {
            ok = false;
            break;
          }
          const uint32_t vf = ptx::smem_u32(&bars->v_full[st]);
          ptx::mbar_arrive_expect_tx(vf, kTileBytes);
          ptx::tma_load_5d(sv + st * kTileBytes, &map_v, vf, 0, (int)(j * kTile), (int)b, (int)(2 * h), 0);
          ptx::tma_load_5d(sv + st * kTileBytes + kBlockBytes, &map_v, vf, 0, (int)(j * kTile), (int)b, (int)(2 * h + 1), 0);
        }
      }
      if (*abort_flag)
        for (uint32_t k = 0; k < (kt < (uint32_t)kT1VStages ? kt : (uint32_t)kT1VStages); ++k) {
          const uint32_t t = kt - 1 - k;
          ptx::mbar_wait_drain(ptx::smem_u32(&bars->v_full[t % kT1VStages]), (t / kT1VStages) & 1, kAttnDrainLimit);
        }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Two cursors walk the CTA's steps (key tiles of its items, in order): one issues scores, up to
    // three steps ahead of the other, which issues P V products as the probabilities arrive.  The
    // score cursor crosses item boundaries, so the first scores of the next query tile are ready
    // when the softmax threads get there.
    if (lane == 0) {
      const uint32_t idesc_s = ptx::idesc_f16_f32(kTile, kTile, 0, 0);        // 128 queries x 128 keys
      const uint32_t idesc_pv = ptx::idesc_f16_f32(kTile, kTile, 0, 1);       // 128 queries x 128 dims, V MN-major
      const uint32_t tg = tmem_base, to = tmem_base + 384;
      auto ready = [&](uint64_t* bar, uint32_t parity) { return ptx::mbar_test_wait(ptx::smem_u32(bar), parity); };
      // first valid item at or after `item`: its step count, or 0 when there is none
      auto seek = [&](uint32_t& item) -> uint32_t {
        for (; item < num_items; item += gridDim.x) {
          uint32_t qt, b, h;
          if (decode_unit_item(P, units, item, qt, b, h)) return qt + 1;
        }
        return 0;
      };
      uint32_t item_s = blockIdx.x, item_p = blockIdx.x;
      uint32_t n_s = seek(item_s), n_p = seek(item_p);
      uint32_t s = 0, p = 0;       // step within the cursor's item
      uint32_t gs = 0, gp = 0;     // steps issued so far by either cursor: ring slots and barrier phases
      uint32_t q_items = 0;        // items whose scores have been started: phase of q_full
      long long t_last = clock64();
      while (n_p != 0) {
        bool progress = false;
        if (n_s != 0 && gs < gp + 3) {
          const uint32_t ks = gs % kT1KStages, sb = gs % 3;
          bool can = ready(&bars->k_full[ks], (gs / kT1KStages) & 1);
          if (can && s == 0) can = ready(&bars->q_full, q_items & 1);
          if (can && gs >= 3)   // the buffer's previous P has been consumed
            can = ready(&bars->pv_done[sb], ((gs - 3) / 3) & 1);
          if (can) {
            ptx::tc_fence_after_sync();
            const uint32_t kb = sk + ks * kTileBytes;
#pragma unroll
            for (int k16 = 0; k16 < kTile / 16; ++k16) {
              const uint32_t off = (k16 >> 2) * kBlockBytes + (k16 & 3) * 32;
              ptx::umma_f16(tg + sb * kTile, ptx::smem_desc_sw128(sq + off, 16, 1024),
                            ptx::smem_desc_sw128(kb + off, 16, 1024), idesc_s, k16 != 0);
            }
            ptx::umma_commit(ptx::smem_u32(&bars->s_full[sb]));
            ptx::umma_commit(ptx::smem_u32(&bars->k_empty[ks]));
            ++gs;
            if (++s == n_s) {   // Q is not read again: the producer may load the next item's
              ptx::umma_commit(ptx::smem_u32(&bars->q_empty));
              ++q_items;
              s = 0;
              item_s += gridDim.x;
              n_s = seek(item_s);
            }
            progress = true;
          }
        }
        if (gp < gs) {
          const uint32_t vs = gp % kT1VStages, sb = gp % 3;
          bool can = ready(&bars->v_full[vs], (gp / kT1VStages) & 1);
#ifdef TSB_TUNING
          if (P.tune_mode != 1)
#endif
          if (can) can = ready(&bars->p_full[sb], (gp / 3) & 1);
          if (can) {
            ptx::tc_fence_after_sync();
            const uint32_t vb = sv + vs * kTileBytes;
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
              const uint64_t db = ptx::smem_desc_sw128(vb + kk * 2048, kBlockBytes, 1024);
              ptx::umma_f16_ts(to, tg + sb * kTile + kk * 8, db, idesc_pv, (p ? 1u : 0u) | (uint32_t)kk);
            }
            ptx::umma_commit(ptx::smem_u32(&bars->pv_done[sb]));
            ptx::umma_commit(ptx::smem_u32(&bars->v_empty[vs]));
            ++gp;
            if (++p == n_p) {
              p = 0;
              item_p += gridDim.x;
              n_p = seek(item_p);
            }
            progress = true;
          }
        }
        if (progress) {
          t_last = clock64();
        } else {
          if (*abort_flag) break;
          if (clock64() - t_last > kAttnWaitLimit) { *abort_flag = 1; break; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax + output: one query row per thread
    const uint32_t quarter = warp & 3;              // TMEM lane quarter this warp may read
    const uint32_t row = quarter * 32 + lane;
    const uint32_t tg = tmem_base + ((quarter * 32u) << 16), to = tg + 384;
    const float c = P.scale_log2;
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait_bounded(ptx::smem_u32(bar), parity, abort_flag,
                                                            kAttnWaitLimit)) != 0;
    };
    uint32_t U = 0;   // steps processed in earlier items
    bool ok = true;
    // The finished item whose output is still in tensor memory.  It is written out after the
    // probabilities of the next item's first step have been computed (the wait for the item's last
    // P V product is hidden behind that arithmetic) and before they are announced: the next item's
    // first P V product overwrites O.
    bool pending = false;
    uint32_t pend_last = 0;          // global index of the pending item's last step
    float pend_inv = 0.f;
    int64_t pend_grow = 0;
    uint32_t pend_h = 0;
    bool pend_row_ok = false;
    auto write_output = [&]() -> bool {
      // the last P V product (MMAs complete in order, so every earlier one has finished too)
      if (!warp_wait(&bars->pv_done[pend_last % 3], (pend_last / 3) & 1)) return false;
      ptx::tc_fence_after_sync();
      uint32_t o[4][32];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) ptx::tmem_ld_32x32(to + ch * 32, o[ch]);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        __half* dst = P.out + (int64_t)(2 * pend_h + (ch >> 1)) * P.stick_stride + pend_grow * kStickHalfs + (ch & 1) * 32;
#pragma unroll
        for (int v = 0; v < 4; v += 2) {
          Vec8h ov[2];
#pragma unroll
          for (int w = 0; w < 2; ++w)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = (v + w) * 8 + 2 * e;
              ov[w].h2[e] = __floats2half2_rn(__uint_as_float(o[ch][i]) * pend_inv, __uint_as_float(o[ch][i + 1]) * pend_inv);
            }
          if (pend_row_ok) ptx::st_global_v8(dst + v * 8, ov[0].u, ov[1].u);   // whole 32-byte sectors
        }
      }
      ptx::tc_fence_before_sync();
      pending = false;
      return true;
    };
#ifdef TSB_TUNING
    long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long prof_start = clock64();
    if (P.tune_mode == 1) ok = false;
#endif
    for (uint32_t item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      uint32_t qt, b, h;
      if (!decode_unit_item(P, units, item, qt, b, h)) continue;
      const uint32_t n = qt + 1;
      float m = -1e30f, l = 0.f;
      for (uint32_t u = 0; u < n; ++u) {
        const uint32_t ug = U + u, buf = ug % 3, ts = tg + buf * kTile;
        bool got_s;
        ATTN_PROF(0, got_s = warp_wait(&bars->s_full[buf], (ug / 3) & 1));
        if (!got_s) { ok = false; break; }
        ptx::tc_fence_after_sync();
        uint32_t r[4][32];
#ifdef TSB_TUNING
        const long long t_ld = clock64();
#endif
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) ptx::tmem_ld_32x32(ts + ch * 32, r[ch]);
        ptx::tmem_ld_wait();
#ifdef TSB_TUNING
        const long long t_max = clock64();
        prof[1] += t_max - t_ld;
#endif
        if (u == qt) {   // diagonal tile: keys after the query do not exist
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if ((uint32_t)(ch * 32 + i) > row) r[ch][i] = 0xff800000u;   // -inf
        }
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(r[ch][i]));
        const float tile_max = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                     fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        if (u == 0) {
          m = tile_max;   // key 0 exists for every query, so this is finite
        } else if (__any_sync(0xffffffffu, (tile_max - m) * c > kRescaleThreshold)) {
          // raise the exponent offset (lazily): O and l shrink by alpha.  O must be at rest: the latest
          // P V product is the one of the previous step.
          if (!warp_wait(&bars->pv_done[(ug - 1) % 3], ((ug - 1) / 3) & 1)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const float m_new = fmaxf(m, tile_max);
          const float alpha = ex2f((m - m_new) * c);
          l *= alpha;
          m = m_new;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[32];
            ptx::tmem_ld_32x32(to + ch * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ptx::tmem_st_32x32(to + ch * 32, o);
          }
          ptx::tmem_st_wait();
        }
        const float mc = m * c;
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#ifdef TSB_TUNING
        const long long t_exp = clock64();
        prof[2] += t_exp - t_max;
#endif
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {   // 64 keys -> 32 packed columns at a time
          uint32_t packed[32];
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = ex2f(fmaf(__uint_as_float(r[hf * 2 + ch][i]), c, -mc));
              const float p1 = ex2f(fmaf(__uint_as_float(r[hf * 2 + ch][i + 1]), c, -mc));
              sum[(i >> 1) & 3] += p0 + p1;
              const __half2 hp = __floats2half2_rn(p0, p1);
              packed[ch * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&hp);
            }
          ptx::tmem_st_32x32(ts + hf * 32, packed);   // P over the scores just read: keys 2c, 2c+1 in column c
        }
        l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
#ifdef TSB_TUNING
        const long long t_st = clock64();
        prof[3] += t_st - t_exp;
#endif
        ptx::tmem_st_wait();
        if (u == 0 && pending) {
#ifdef TSB_TUNING
          const long long t_fin = clock64();
#endif
          if (!write_output()) { ok = false; break; }
#ifdef TSB_TUNING
          prof[5] += clock64() - t_fin;
#endif
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->p_full[buf]));
#ifdef TSB_TUNING
        prof[4] += clock64() - t_st;
#endif
      }
      if (!ok) break;
      U += n;
      pending = true;
      pend_last = U - 1;
      pend_inv = 1.f / l;
      pend_row_ok = qt * kTile + row < P.seq;
      pend_grow = (int64_t)b * P.seq + (int64_t)qt * kTile + row;
      pend_h = h;
    }
    if (ok && pending) {
#ifdef TSB_TUNING
      const long long t_fin = clock64();
#endif
      write_output();
#ifdef TSB_TUNING
      prof[5] += clock64() - t_fin;
#endif
    }
#ifdef TSB_TUNING
    if (warp == 2 && lane == 0) {
      for (int i = 0; i < 6; ++i) atomicAdd(&g_attn_prof[i], (unsigned long long)prof[i]);
      atomicAdd(&g_attn_prof[7], (unsigned long long)(clock64() - prof_start));
    }
#endif
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kAttnTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) atomicExch(&g_attn_error, 1);
}

int g_attn_sm_count = 0;

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_attention_causal_f16(const void* q, const void* k, const void* v, void* out,
                                       int64_t batch, int64_t seq, int64_t heads, int64_t head_dim,
                                       float scale, void* stream) {
  if (batch < 0 || seq < 0 || heads < 0) return TS_ERR_INVALID;
  if (batch == 0 || seq == 0 || heads == 0) return TS_OK;
  if (!q || !k || !v || !out) return TS_ERR_INVALID;
  if (head_dim != kTile) return TS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) % 128) return TS_ERR_ALIGNMENT;
  if (!(scale > 0.f)) return TS_ERR_INVALID;
  // A last tile that runs past seq reads zeros there (the tensor map has seq as its own dim);
  // the causal mask already hides those keys from every real query, and their rows are not stored.
  const int64_t rows = batch * seq, q_tiles = ceil_div(seq, (int64_t)kTile);
  const int64_t items = q_tiles * batch * heads;
  if (rows >= (1ll << 31) || items >= (1ll << 31) || heads * 2 >= (1ll << 31)) return TS_ERR_TOO_LARGE;
  AttnParams P{};
  P.out = (__half*)out;
  P.batch = (uint32_t)batch; P.seq = (uint32_t)seq; P.heads = (uint32_t)heads;
  P.q_tiles = (uint32_t)q_tiles; P.num_items = (uint32_t)items;
  P.stick_stride = rows * kStickHalfs;
  P.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap mq, mk, mv;
  if (!make_stick_map(&mq, q, (uint64_t)seq, (uint64_t)batch, (uint64_t)(2 * heads), 1, P.stick_stride, 0, kTile) ||
      !make_stick_map(&mk, k, (uint64_t)seq, (uint64_t)batch, (uint64_t)(2 * heads), 1, P.stick_stride, 0, kTile) ||
      !make_stick_map(&mv, v, (uint64_t)seq, (uint64_t)batch, (uint64_t)(2 * heads), 1, P.stick_stride, 0, kTile))
    return TS_ERR_CUDA;
  if (g_attn_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_attn_sm_count = n;
  }
#ifdef TSB_TUNING
  P.tune_mode = getenv("TS_ATTN_MODE") ? atoi(getenv("TS_ATTN_MODE")) : 0;
#endif
  int which_kernel = 0;   // 0: by shape
#ifdef TSB_TUNING
  if (getenv("TS_ATTN_KERNEL")) which_kernel = atoi(getenv("TS_ATTN_KERNEL"));
#endif
  if (q_tiles % 2 != 0 || which_kernel == 3) {
    // one query tile per CTA
    const int64_t sms = g_attn_sm_count > 0 ? g_attn_sm_count : 148;
    P.heads_per_round = (uint32_t)std::min<int64_t>(sms / q_tiles, batch * heads);
    const uint32_t grid1 = (uint32_t)std::min<int64_t>(items, sms);
    const cudaError_t e3 = cudaFuncSetAttribute(attention_causal_tmem_kernel,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kT1Smem);
    if (e3 != cudaSuccess) { note_cuda_error(e3); return TS_ERR_CUDA; }
    attention_causal_tmem_kernel<<<grid1, kT1Threads, kT1Smem, (cudaStream_t)stream>>>(mq, mk, mv, P);
    TSB_CHECK_LAUNCH();
    return TS_OK;
  }
  if (q_tiles % 2 == 0) {
    // two query tiles per CTA
    const int64_t pair_items = items / 2, pairs = q_tiles / 2;
    const int64_t sms = g_attn_sm_count > 0 ? g_attn_sm_count : 148;
    P.heads_per_round = (uint32_t)std::min<int64_t>(sms / pairs, batch * heads);
    // every SM gets a CTA: those beyond heads_per_round * pairs are the spares of pair_layout()
    const uint32_t grid2 = (uint32_t)std::min<int64_t>(pair_items, sms);
    const cudaError_t e2 = cudaFuncSetAttribute(attention_causal_pair64_kernel,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kP64Smem);
    if (e2 != cudaSuccess) { note_cuda_error(e2); return TS_ERR_CUDA; }
    attention_causal_pair64_kernel<<<grid2, kPairAttnThreads, kP64Smem, (cudaStream_t)stream>>>(mq, mk, mv, P);
    TSB_CHECK_LAUNCH();
    return TS_OK;
  }
  return TS_ERR_UNSUPPORTED;   // not reached: every tile count is served above
}

// Synchronises the device and reports (and clears) the sticky error word the attention kernel
// sets when one of its bounded waits gave up.  Returns 0, 1 or an error code.
extern "C" int ts_attention_error_state(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return TS_ERR_CUDA;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  }
  return v;
}

#ifdef TSB_TUNING
// tuning build only: reads and clears the experiment counters
extern "C" int ts_attn_prof(unsigned long long* out8) {
  if (cudaMemcpyFromSymbol(out8, g_attn_prof, sizeof(unsigned long long) * 8) != cudaSuccess) return TS_ERR_CUDA;
  unsigned long long zero[8] = {0};
  cudaMemcpyToSymbol(g_attn_prof, zero, sizeof(zero));
  return TS_OK;
}
#endif
