// Stick relayout: strided raw image of a host tensor <-> SpyreTensorLayout stick image.
//
// Stands in for the SenDataConvert host pass of the reference's copy path
// (torch_spyre/csrc/spyre_mem.cpp:213-279).  Like the reference's
// data_conversion_stride_info, the work is described as an iteration space with
// one (size, source stride, destination stride) triple per device dim; the
// planner below builds it from the layout, merges dims that are contiguous on
// both sides and picks one of two kernels:
//   * copy_tiles       - both sides share the unit-stride dim: 16-byte (or
//                        narrower) units are moved as they are, in tiles shaped
//                        so that reads and writes both form long segments;
//   * transpose_tiles  - the unit-stride dims differ (a permuted host tensor):
//                        64x64 fp16 tiles are transposed through shared memory.
#include <algorithm>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <sys/mman.h>

#include "common.cuh"

namespace tsb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnitsPerThread = 8;
constexpr int kMaxChecks = 2;

// Plan dims are stored innermost first: copy_tiles uses dim 0 = the unit-stride run,
// dim 1 = the dim next-most contiguous in the source, dim 2 = next-most contiguous
// in the destination (extent-1 dummies when absent); transpose_tiles uses dim 0 =
// unit stride in the source, dim 1 = unit stride in the destination.
struct CopyPlan {
  int nd;
  uint32_t size[kMaxDims];       // extent per dim (copy_tiles dim 0: in units)
  int64_t sbytes[kMaxDims];      // source stride per dim, bytes
  int64_t dbytes[kMaxDims];      // destination stride per dim, bytes
  uint32_t tile[kMaxDims];       // CTA tile extent per dim (1 = not tiled)
  FastDiv ntiles[kMaxDims];      // tiles per dim
  // Padding: index is inside the host tensor iff, for every check c,
  // sum_d idx[d] * vmul[c][d] < vlimit[c].
  int nchecks;
  int64_t vmul[kMaxChecks][kMaxDims];
  int64_t vlimit[kMaxChecks];
  // kPerCheck mode: an index that fails check c is written as zero when vfill[c] (it is a pad
  // lane of the destination image) and skipped otherwise (it does not exist in the destination)
  int vfill[kMaxChecks];
  // copy_tiles: 256 threads cover T0 x T1 x T2 indices of dims 0,1,2; each thread then
  // walks kUnitsPerThread steps of `kstep` indices along dim `kd`.
  int log_t0, log_t1, kd;
  uint32_t kstep;
  // transpose_tiles: the plan dim the CTA walks its kSubTiles tiles along: dim 0 or 1 (64 indices
  // per step) or an outer dim (one index per step)
  int sub_dim;
};

// What happens to an index that fails a padding check.
enum FillMode { kSkip = 0 /* image -> strided memory */, kFill = 1 /* strided memory -> image */,
                kPerCheck = 2 /* image -> image: CopyPlan::vfill decides */ };

template <int UNIT>
struct UnitType;
template <> struct UnitType<16> { using T = uint4; };
template <> struct UnitType<8> { using T = uint2; };
template <> struct UnitType<4> { using T = uint32_t; };
template <> struct UnitType<2> { using T = uint16_t; };
template <> struct UnitType<1> { using T = uint8_t; };

template <class T> __device__ __forceinline__ T zero_of() { return T(0); }
template <> __device__ __forceinline__ uint4 zero_of<uint4>() { return make_uint4(0, 0, 0, 0); }
template <> __device__ __forceinline__ uint2 zero_of<uint2>() { return make_uint2(0, 0); }

template <class T> __device__ __forceinline__ T load_unit(const char* p) {
  return *reinterpret_cast<const T*>(p);
}
template <> __device__ __forceinline__ uint4 load_unit<uint4>(const char* p) { return ld_stream_v4(p); }

struct TileBase {
  uint32_t o0, o1, o2;       // tile origin along dims 0, 1, 2
  uint32_t osub;             // tile origin along CopyPlan::sub_dim (transpose_tiles)
  int64_t soff, doff;        // byte offsets of the tile origin
  int64_t v[kMaxChecks];     // check sums at the tile origin
};

template <bool CHECKS>
__device__ __forceinline__ TileBase decode_tile(const CopyPlan& p, uint32_t tile_id) {
  TileBase b;
  b.o0 = b.o1 = b.o2 = b.osub = 0;
  b.soff = b.doff = 0;
  b.v[0] = b.v[1] = 0;
  uint32_t rem = tile_id;
#pragma unroll
  for (int d = 0; d < kMaxDims; ++d) {
    if (d >= p.nd) break;
    uint32_t q, r;
    p.ntiles[d].divmod(rem, q, r);
    rem = q;
    const uint32_t o = r * p.tile[d];
    if (d == 0) b.o0 = o;
    if (d == 1) b.o1 = o;
    if (d == 2) b.o2 = o;
    if (d == p.sub_dim) b.osub = o;
    b.soff += (int64_t)o * p.sbytes[d];
    b.doff += (int64_t)o * p.dbytes[d];
    if (CHECKS) {
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c) b.v[c] += (int64_t)o * p.vmul[c][d];
    }
  }
  return b;
}

// ---------------------------------------------------------------------------
template <int UNIT, int MODE, bool CHECKS>
__global__ void __launch_bounds__(kThreads)
copy_tiles(const __grid_constant__ CopyPlan p, const char* __restrict__ src, char* __restrict__ dst) {
  using T = typename UnitType<UNIT>::T;
  const TileBase b = decode_tile<CHECKS>(p, blockIdx.x);
  const uint32_t t = threadIdx.x;
  const uint32_t i0 = t & ((1u << p.log_t0) - 1);
  const uint32_t i1 = (t >> p.log_t0) & ((1u << p.log_t1) - 1);
  const uint32_t i2 = t >> (p.log_t0 + p.log_t1);
  const uint32_t x0 = b.o0 + i0, x1 = b.o1 + i1, x2 = b.o2 + i2;
  const char* sp = src + b.soff + (int64_t)i0 * p.sbytes[0] + (int64_t)i1 * p.sbytes[1] +
                   (int64_t)i2 * p.sbytes[2];
  char* dp = dst + b.doff + (int64_t)i0 * p.dbytes[0] + (int64_t)i1 * p.dbytes[1] +
             (int64_t)i2 * p.dbytes[2];
  int64_t vv[kMaxChecks] = {0, 0};
  if (CHECKS) {
#pragma unroll
    for (int c = 0; c < kMaxChecks; ++c)
      vv[c] = b.v[c] + (int64_t)i0 * p.vmul[c][0] + (int64_t)i1 * p.vmul[c][1] +
              (int64_t)i2 * p.vmul[c][2];
  }
  // the dim the k loop walks, its current index and the per-step deltas
  const int kd = p.kd;
  uint32_t xk = kd == 0 ? x0 : (kd == 1 ? x1 : x2);
  const uint32_t nk = p.size[kd];
  const bool fixed_ok = (kd == 0 || x0 < p.size[0]) && (kd == 1 || x1 < p.size[1]) &&
                        (kd == 2 || x2 < p.size[2]);
  const int64_t ds = (int64_t)p.kstep * p.sbytes[kd], dd = (int64_t)p.kstep * p.dbytes[kd];
  int64_t dv[kMaxChecks] = {0, 0};
  if (CHECKS) {
#pragma unroll
    for (int c = 0; c < kMaxChecks; ++c) dv[c] = (int64_t)p.kstep * p.vmul[c][kd];
  }
  T val[kUnitsPerThread];
  bool live[kUnitsPerThread];
#pragma unroll
  for (int k = 0; k < kUnitsPerThread; ++k) {
    const bool inb = fixed_ok && (xk + k * p.kstep < nk);
    bool valid = true, exists = true;
    if (CHECKS) {
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c)
        if (c < p.nchecks) {
          const bool ok = vv[c] + k * dv[c] < p.vlimit[c];
          valid = valid && ok;
          if (MODE == kSkip || (MODE == kPerCheck && !p.vfill[c])) exists = exists && ok;
        }
    }
    val[k] = zero_of<T>();
    if (inb && valid) val[k] = load_unit<T>(sp + k * ds);
    live[k] = inb && exists;
  }
#pragma unroll
  for (int k = 0; k < kUnitsPerThread; ++k)
    if (live[k]) *reinterpret_cast<T*>(dp + k * dd) = val[k];
}

// ---------------------------------------------------------------------------
// 64x64 tiles of 2-byte elements; a CTA takes kSubTiles of them along the longer of
// dims 0 and 1.  smem holds a tile as [row = dim-1 index][col = dim-0 index], 32-bit words, pitch 33 words
// so that both phases are free of bank conflicts.
constexpr int kTT = 64;
constexpr int kSubTiles = 4;
constexpr int kPitchWords = 33;

// Number of leading elements (0..8), along dim `dim`, that satisfy every check, given
// the check sums at the first element.
template <bool ONLY_SKIPPING = false>
__device__ __forceinline__ int valid_run(const CopyPlan& p, const int64_t* vsum, int dim) {
  int n = 8;
#pragma unroll
  for (int c = 0; c < kMaxChecks; ++c) {
    if (c < p.nchecks && !(ONLY_SKIPPING && p.vfill[c])) {
      const int64_t room = p.vlimit[c] - vsum[c];
      const int64_t mul = p.vmul[c][dim];
      int64_t k;
      if (room <= 0) k = 0;
      else if (mul == 0) k = 8;
      else k = (room + mul - 1) / mul;
      n = (int)(k < n ? k : n);
    }
  }
  return n;
}

template <int MODE, bool VEC_IN, bool VEC_OUT, bool CHECKS>
__global__ void __launch_bounds__(kThreads, 4)
transpose_tiles(const __grid_constant__ CopyPlan p, const char* __restrict__ src,
                char* __restrict__ dst) {
  __shared__ uint32_t tile[kSubTiles][kTT * kPitchWords];
  const TileBase b = decode_tile<CHECKS>(p, blockIdx.x);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sd = p.sub_dim;
  // phase 1 role: row (dim 1) and 16-byte vector (dim 0)
  const int row1 = threadIdx.x >> 3, vec1 = threadIdx.x & 7;
  // phase 2 role: word column (two dim-0 indices) and group of 8 dim-1 indices
  const int pcol = 8 * (warp & 3) + (lane & 7);
  const int grp = 4 * (warp >> 2) + (lane >> 3);
  const char* sp0 = src + b.soff + (int64_t)row1 * p.sbytes[1] + vec1 * 16;
  const int64_t srow32 = 32 * p.sbytes[1];
  char* dp0 = dst + b.doff + (int64_t)(2 * pcol) * p.dbytes[0] + grp * 16;
  // byte and index steps from one sub-tile to the next
  const int sub_idx = sd < 2 ? kTT : 1;
  const int64_t sub_s = (int64_t)sub_idx * p.sbytes[sd], sub_d = (int64_t)sub_idx * p.dbytes[sd];
  const int step_a = sd == 0 ? kTT : 0, step_b = sd == 1 ? kTT : 0;
  // extent left in this CTA's first sub-tile (may exceed one tile)
  const int left_a = (int)(p.size[0] - b.o0), left_b = (int)(p.size[1] - b.o1);
  // sub-tiles that exist when they are walked along an outer dim
  const int left_sub = sd < 2 ? kSubTiles : (int)(p.size[sd] - b.osub);

  // Phase 1: every load of the CTA's sub-tiles is issued before the first use, so the
  // sub-tiles' rows (adjacent in memory when they lie along dim 0) reach DRAM together.
  uint32_t w[kSubTiles][2][4];
#pragma unroll
  for (int sub = 0; sub < kSubTiles; ++sub) {
    const int rem_a = left_a - sub * step_a, rem_b = left_b - sub * step_b;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int row = row1 + k * 32;
      int na = rem_a - vec1 * 8;
      na = na < 0 ? 0 : (na > 8 ? 8 : na);
      if (row >= rem_b || sub >= left_sub) na = 0;
      if (CHECKS && MODE != kSkip && na > 0) {
        int64_t vs[kMaxChecks];
#pragma unroll
        for (int c = 0; c < kMaxChecks; ++c)
          vs[c] = b.v[c] + (int64_t)(sub * step_b + row) * p.vmul[c][1] +
                  (int64_t)(sub * step_a + vec1 * 8) * p.vmul[c][0] +
                  (sd < 2 ? 0 : (int64_t)sub * p.vmul[c][sd]);
        na = min(na, valid_run(p, vs, 0));
      }
      const char* sp = sp0 + k * srow32 + sub * sub_s;
      uint32_t(&q)[4] = w[sub][k];
      q[0] = q[1] = q[2] = q[3] = 0;
      if (VEC_IN && na == 8) {
        const uint4 v = ld_stream_v4(sp);
        q[0] = v.x; q[1] = v.y; q[2] = v.z; q[3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < na) {
            const uint32_t e = *reinterpret_cast<const uint16_t*>(sp + 2 * j);
            q[j >> 1] |= e << ((j & 1) * 16);
          }
        }
      }
    }
  }
#pragma unroll
  for (int sub = 0; sub < kSubTiles; ++sub) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint32_t* tp = &tile[sub][(row1 + k * 32) * kPitchWords + vec1 * 4];
      tp[0] = w[sub][k][0]; tp[1] = w[sub][k][1]; tp[2] = w[sub][k][2]; tp[3] = w[sub][k][3];
    }
  }
  __syncthreads();

  // Phase 2: output rows along dim 0 (two per thread), 8 consecutive dim-1 indices each.
#pragma unroll
  for (int sub = 0; sub < kSubTiles; ++sub) {
    const int rem_a = left_a - sub * step_a, rem_b = left_b - sub * step_b;
    uint32_t t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = tile[sub][(8 * grp + j) * kPitchWords + pcol];
    int nb = rem_b - grp * 8;
    nb = nb < 0 ? 0 : (nb > 8 ? 8 : nb);
    if (sub >= left_sub) nb = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int a = 2 * pcol + half;
      if (a >= rem_a) continue;
      int n = nb;
      if (CHECKS && MODE != kFill && n > 0) {
        int64_t vs[kMaxChecks];
#pragma unroll
        for (int c = 0; c < kMaxChecks; ++c)
          vs[c] = b.v[c] + (int64_t)(sub * step_a + a) * p.vmul[c][0] +
                  (int64_t)(sub * step_b + grp * 8) * p.vmul[c][1] +
                  (sd < 2 ? 0 : (int64_t)sub * p.vmul[c][sd]);
        n = min(n, valid_run<MODE == kPerCheck>(p, vs, 1));
      }
      const uint32_t sel = half ? 0x7632u : 0x5410u;
      uint4 q;
      q.x = __byte_perm(t[0], t[1], sel);
      q.y = __byte_perm(t[2], t[3], sel);
      q.z = __byte_perm(t[4], t[5], sel);
      q.w = __byte_perm(t[6], t[7], sel);
      char* dp = dp0 + sub * sub_d + (int64_t)half * p.dbytes[0];
      if (VEC_OUT && n == 8) {
        st_global_v4(dp, q);
      } else {
        const uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < n) *reinterpret_cast<uint16_t*>(dp + 2 * j) = (uint16_t)(ww[j >> 1] >> ((j & 1) * 16));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host-side planner.

struct IterDim {
  int64_t size, s, d;          // strides in elements
  int64_t vm[kMaxChecks];
};

int log2_floor(uint32_t x) {
  int l = 0;
  while ((2u << l) <= x) ++l;
  return l;
}
uint32_t pow2_ceil(uint32_t x) {
  uint32_t p = 1;
  while (p < x) p <<= 1;
  return p;
}

struct Request {
  const char* src;
  char* dst;
  bool to_device;
  int elem_bytes;
  const int64_t *host_size, *host_strides;
  int rank;
  const int64_t *dev_size, *dev_strides;
  const int32_t* dim_map;
  int ndev;
};

template <int MODE, bool CHECKS>
int launch_copy2(const CopyPlan& plan, int unit, uint32_t blocks, const char* src, char* dst,
                 cudaStream_t st) {
  switch (unit) {
    case 16: copy_tiles<16, MODE, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 8: copy_tiles<8, MODE, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 4: copy_tiles<4, MODE, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 2: copy_tiles<2, MODE, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    default: copy_tiles<1, MODE, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
  }
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
int launch_copy(const CopyPlan& plan, int mode, int unit, bool checks, uint32_t blocks, const char* src,
                char* dst, cudaStream_t st) {
  if (!checks)   // without checks the mode makes no difference
    return launch_copy2<kFill, false>(plan, unit, blocks, src, dst, st);
  if (mode == kFill) return launch_copy2<kFill, true>(plan, unit, blocks, src, dst, st);
  if (mode == kSkip) return launch_copy2<kSkip, true>(plan, unit, blocks, src, dst, st);
  return launch_copy2<kPerCheck, true>(plan, unit, blocks, src, dst, st);
}

template <int MODE, bool CHECKS>
int launch_transpose2(const CopyPlan& plan, bool vin, bool vout, uint32_t blocks, const char* src,
                      char* dst, cudaStream_t st) {
  if (vin && vout) transpose_tiles<MODE, true, true, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else if (vin) transpose_tiles<MODE, true, false, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else if (vout) transpose_tiles<MODE, false, true, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else transpose_tiles<MODE, false, false, CHECKS><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}
int launch_transpose(const CopyPlan& plan, int mode, bool vin, bool vout, bool checks, uint32_t blocks,
                     const char* src, char* dst, cudaStream_t st) {
  if (!checks) return launch_transpose2<kFill, false>(plan, vin, vout, blocks, src, dst, st);
  if (mode == kFill) return launch_transpose2<kFill, true>(plan, vin, vout, blocks, src, dst, st);
  if (mode == kSkip) return launch_transpose2<kSkip, true>(plan, vin, vout, blocks, src, dst, st);
  return launch_transpose2<kPerCheck, true>(plan, vin, vout, blocks, src, dst, st);
}

int plan_and_launch(IterDim* it, int nd, int nchecks, const int64_t* vlimit, const int* vfill, int mode,
                    int eb, const char* src, char* dst, cudaStream_t st);

int run(const Request& rq, cudaStream_t st) {
  if (!rq.host_size || !rq.host_strides || !rq.dev_size || !rq.dev_strides || !rq.dim_map)
    return TS_ERR_INVALID;
  if (rq.rank < 1 || rq.rank > kMaxDims || rq.ndev < 1 || rq.ndev > kMaxDims) return TS_ERR_INVALID;
  if (rq.elem_bytes != 1 && rq.elem_bytes != 2 && rq.elem_bytes != 4 && rq.elem_bytes != 8) return TS_ERR_INVALID;
  const int eb = rq.elem_bytes;
  int64_t total = 1;
  for (int d = 0; d < rq.ndev; ++d) {
    if (rq.dev_size[d] < 0 || rq.dim_map[d] < 0 || rq.dim_map[d] >= rq.rank) return TS_ERR_INVALID;
    total *= rq.dev_size[d];
  }
  for (int h = 0; h < rq.rank; ++h) {
    if (rq.host_size[h] < 0) return TS_ERR_INVALID;
    if (rq.host_size[h] == 0 && !rq.to_device) return TS_OK;
  }
  if (total == 0) return TS_OK;
  if (!rq.src || !rq.dst) return TS_ERR_INVALID;

  // One iteration dim per device dim.  A host dim mapped by several device dims
  // is split over them, outermost most significant.
  IterDim it[kMaxDims];
  int nchecks = 0;
  int64_t vlimit[kMaxChecks] = {0, 0};
  int check_of_host[kMaxDims];
  for (int h = 0; h < rq.rank; ++h) {
    check_of_host[h] = -1;
    int64_t cover = 1;
    bool mapped = false;
    for (int d = 0; d < rq.ndev; ++d)
      if (rq.dim_map[d] == h) { cover *= rq.dev_size[d]; mapped = true; }
    if (!mapped) {
      if (rq.host_size[h] != 1) return TS_ERR_INVALID;
      continue;
    }
    if (cover < rq.host_size[h]) return TS_ERR_INVALID;
    if (cover > rq.host_size[h]) {
      if (nchecks == kMaxChecks) return TS_ERR_UNSUPPORTED;
      check_of_host[h] = nchecks;
      vlimit[nchecks++] = rq.host_size[h];
    }
  }
  for (int d = 0; d < rq.ndev; ++d) {
    const int h = rq.dim_map[d];
    int64_t mult = 1;
    for (int e = rq.ndev - 1; e > d; --e)
      if (rq.dim_map[e] == h) mult *= rq.dev_size[e];
    const int64_t host_step = mult * rq.host_strides[h];
    it[d].size = rq.dev_size[d];
    it[d].s = rq.to_device ? host_step : rq.dev_strides[d];
    it[d].d = rq.to_device ? rq.dev_strides[d] : host_step;
    for (int c = 0; c < kMaxChecks; ++c) it[d].vm[c] = (check_of_host[h] == c) ? mult : 0;
  }
  const int fill[kMaxChecks] = {rq.to_device ? 1 : 0, rq.to_device ? 1 : 0};
  return plan_and_launch(it, rq.ndev, nchecks, vlimit, fill, rq.to_device ? kFill : kSkip, eb, rq.src,
                         rq.dst, st);
}

// Turns an iteration space into a CopyPlan and launches the kernel that suits it.  `it` has room
// for kMaxDims entries and is modified.
int plan_and_launch(IterDim* it, int nd_in, int nchecks, const int64_t* vlimit, const int* vfill, int mode,
                    int eb, const char* src, char* dst, cudaStream_t st) {
  // Drop size-1 dims, then merge neighbours that are contiguous on both sides.
  int nd = 0;
  for (int d = 0; d < nd_in; ++d)
    if (it[d].size != 1) it[nd++] = it[d];
  if (nd == 0) { it[0] = IterDim{1, 1, 1, {0, 0}}; nd = 1; }
  for (int d = nd - 2; d >= 0; --d) {
    const IterDim& in = it[d + 1];
    bool ok = it[d].s == in.s * in.size && it[d].d == in.d * in.size;
    for (int c = 0; c < kMaxChecks; ++c) ok = ok && it[d].vm[c] == in.vm[c] * in.size;
    if (ok) {
      it[d + 1].size *= it[d].size;
      for (int e = d; e < nd - 1; ++e) it[e] = it[e + 1];
      --nd;
    }
  }
  for (int d = 0; d < nd; ++d)
    if (it[d].size >= (1ll << 31)) return TS_ERR_TOO_LARGE;

  CopyPlan plan{};
  plan.nchecks = nchecks;
  for (int c = 0; c < kMaxChecks; ++c) {
    plan.vlimit[c] = vlimit[c];
    plan.vfill[c] = vfill[c];
  }
  const bool checks = nchecks > 0;

  int ua = -1, ub = -1;  // unit-stride dims of source / destination
  for (int d = 0; d < nd; ++d) {
    if (it[d].s == 1 && ua < 0) ua = d;
    if (it[d].d == 1 && ub < 0) ub = d;
  }
  const uintptr_t sbase = (uintptr_t)src, dbase = (uintptr_t)dst;

  // Fills plan dims from `order` (plan position -> index into it[]); unit = bytes per
  // index step of plan dim 0 on the copy path (elements there are grouped into units).
  auto fill = [&](const int* order, int n, int unit_elems) {
    plan.nd = n;
    for (int k = 0; k < n; ++k) {
      const IterDim& d = it[order[k]];
      const bool grouped = k == 0 && unit_elems > 1;
      plan.size[k] = (uint32_t)(grouped ? d.size / unit_elems : d.size);
      plan.sbytes[k] = d.s * eb * (grouped ? unit_elems : 1);
      plan.dbytes[k] = d.d * eb * (grouped ? unit_elems : 1);
      for (int c = 0; c < kMaxChecks; ++c) plan.vmul[c][k] = d.vm[c] * (grouped ? unit_elems : 1);
      plan.tile[k] = 1;
    }
  };
  auto count_tiles = [&](uint64_t& ntiles) {
    ntiles = 1;
    for (int k = 0; k < plan.nd; ++k) {
      const uint32_t nt = (uint32_t)ceil_div(plan.size[k], plan.tile[k]);
      plan.ntiles[k].init(nt);
      ntiles *= nt;
    }
    return ntiles < (1ull << 31);
  };

  if (eb == 2 && ua >= 0 && ub >= 0 && ua != ub && it[ua].size >= 16 && it[ub].size >= 16) {
    // ---- transpose path: plan dim 0 = source-contiguous, dim 1 = destination-contiguous
    int order[kMaxDims], n = 0;
    order[n++] = ua;
    order[n++] = ub;
    for (int d = nd - 1; d >= 0; --d)
      if (d != ua && d != ub) order[n++] = d;
    fill(order, n, 1);
    bool vin = sbase % 16 == 0, vout = dbase % 16 == 0;
    for (int k = 0; k < n; ++k) {
      if (k != 0 && plan.sbytes[k] % 16) vin = false;
      if (k != 1 && plan.dbytes[k] % 16) vout = false;
    }
    // The CTA's kSubTiles tiles lie along the longer tiled dim, or, when neither has room for
    // them (a transpose between two stick images: both are one stick wide), along the outer dim
    // whose steps are closest together in the source, so that the tiles' rows are neighbours in
    // memory and reach DRAM together.
    plan.sub_dim = plan.size[0] >= plan.size[1] ? 0 : 1;
    if (plan.size[plan.sub_dim] < (uint32_t)(2 * kTT)) {
      int best = -1;
      for (int k = 2; k < n; ++k)
        if (plan.size[k] > 1 && plan.sbytes[k] > 0 && (best < 0 || plan.sbytes[k] < plan.sbytes[best])) best = k;
      if (best >= 0) plan.sub_dim = best;
    }
    plan.tile[0] = kTT * (plan.sub_dim == 0 ? kSubTiles : 1);
    plan.tile[1] = kTT * (plan.sub_dim == 1 ? kSubTiles : 1);
    if (plan.sub_dim >= 2) plan.tile[plan.sub_dim] = kSubTiles;
    uint64_t ntiles;
    if (!count_tiles(ntiles)) return TS_ERR_TOO_LARGE;
    return launch_transpose(plan, mode, vin, vout, checks, (uint32_t)ntiles, src, dst, st);
  }

  // ---- copy path.  Plan dim 0 must have unit stride on both sides; an extent-1 dummy
  // stands in when the tensor has none.
  int inner = -1;
  for (int d = 0; d < nd; ++d)
    if (it[d].s == 1 && it[d].d == 1) inner = d;
  if (inner < 0) {
    if (nd == kMaxDims) return TS_ERR_UNSUPPORTED;
    it[nd] = IterDim{1, 1, 1, {0, 0}};
    inner = nd++;
  }
  // Widest unit (bytes) dividing every address, the inner extent and the limits.
  int unit = 16;
  auto fits = [&](int u) {
    if (u < eb) return false;
    if (u == eb) return true;
    const int ue = u / eb;
    if (sbase % u || dbase % u) return false;
    if (it[inner].size % ue) return false;
    for (int d = 0; d < nd; ++d)
      if (d != inner && ((it[d].s * eb) % u || (it[d].d * eb) % u)) return false;
    for (int c = 0; c < nchecks; ++c)
      if (it[inner].vm[c] != 0 && vlimit[c] % ue) return false;
    return true;
  };
  while (!fits(unit)) unit >>= 1;
  // dims next-most contiguous in the source (dx) and in the destination (dy)
  int dx = -1, dy = -1;
  for (int d = 0; d < nd; ++d) {
    if (d == inner) continue;
    if (dx < 0 || llabs(it[d].s) < llabs(it[dx].s)) dx = d;
  }
  for (int d = 0; d < nd; ++d) {
    if (d == inner || d == dx) continue;
    if (dy < 0 || llabs(it[d].d) < llabs(it[dy].d)) dy = d;
  }
  // extent-1 dummies keep dims 1 and 2 present
  int extra = nd;
  IterDim dummy{1, 0, 0, {0, 0}};
  if (dx < 0) { if (extra == kMaxDims) return TS_ERR_UNSUPPORTED; it[extra] = dummy; dx = extra++; }
  if (dy < 0) { if (extra == kMaxDims) return TS_ERR_UNSUPPORTED; it[extra] = dummy; dy = extra++; }
  int order[kMaxDims], n = 0;
  order[n++] = inner;
  order[n++] = dx;
  order[n++] = dy;
  for (int d = nd - 1; d >= 0; --d)
    if (d != inner && d != dx && d != dy) order[n++] = d;
  fill(order, n, unit / eb);
  // Thread tile T0 x T1 x T2 = 256 threads; the k loop extends the CTA tile along kd.
  const uint32_t t0 = std::min<uint32_t>(pow2_ceil(plan.size[0]), kThreads);
  const uint32_t rest = kThreads / t0;
  uint32_t t1, t2;
  if (plan.size[2] > 1) {
    const uint32_t want = 1u << ((log2_floor(rest) + 1) / 2);
    t1 = std::min<uint32_t>(want, pow2_ceil(plan.size[1]));
    t2 = rest / t1;
  } else {
    t1 = rest;
    t2 = 1;
  }
  plan.log_t0 = log2_floor(t0);
  plan.log_t1 = log2_floor(t1);
  const int kd = plan.size[2] > 1 ? 2 : (plan.size[1] > t1 ? 1 : 0);
  plan.kd = kd;
  plan.kstep = kd == 2 ? t2 : (kd == 1 ? t1 : t0);
  plan.tile[0] = t0;
  plan.tile[1] = t1;
  plan.tile[2] = t2;
  plan.tile[kd] *= kUnitsPerThread;
  uint64_t ntiles;
  if (!count_tiles(ntiles)) return TS_ERR_TOO_LARGE;
  return launch_copy(plan, mode, unit, checks, (uint32_t)ntiles, src, dst, st);
}

// ---------------------------------------------------------------------------
// Stick image -> stick image for a strided view on either side.
//
// A side is the generic stick image of a row-major base tensor plus a view of that base (sizes
// shared by both sides, element strides and an element offset in the base's row-major numbering):
// what a transposed, permuted, sliced, narrowed or expanded `spyre` tensor is.  The view is
// expressible when every view dim walks along a single base dim, and the dim walking the base's
// innermost (stick) dim does so with step 1 from a stick boundary (or stays inside one stick).
struct ViewSide {
  const int64_t* base;     // row-major base shape
  int nb;
  const int64_t* strides;  // view strides, elements of the base
  int64_t offset;
};

struct SideDim {            // how one view dim moves through a side's stick image
  bool split;              // walks the stick dim across sticks: index = 64 * hi + lo
  int64_t step;            // elements of the image per index (per lo index when split)
  int64_t hi_step;         // elements of the image per stick (split only)
};

// Fills dims[] for every view dim and returns the constant element offset into the image, or a
// negative status.
int64_t decompose_side(const ViewSide& v, const int64_t* size, int rank, int lanes, bool is_dst,
                       SideDim* dims, bool* walks_stick_to_end) {
  if (v.nb < 1 || v.nb + 1 > kMaxDims) return TS_ERR_INVALID;
  int64_t rm[kMaxDims], img[kMaxDims];   // row-major strides of the base; image strides of its dims
  int64_t numel = 1;
  for (int b = v.nb - 1; b >= 0; --b) {
    if (v.base[b] <= 0) return TS_ERR_INVALID;
    rm[b] = numel;
    numel *= v.base[b];
  }
  const int last = v.nb - 1;
  int64_t rows = 1;
  for (int b = last - 1; b >= 0; --b) {
    img[b] = rows * lanes;
    rows *= v.base[b];
  }
  const int64_t stick_stride = rows * lanes;   // between stick columns
  if (v.offset < 0 || v.offset >= numel) return TS_ERR_INVALID;
  int64_t o[kMaxDims];
  for (int b = 0; b < v.nb; ++b) o[b] = (v.offset / rm[b]) % v.base[b];
  bool used[kMaxDims] = {false};
  int64_t constant = 0;
  for (int b = 0; b < last; ++b) constant += o[b] * img[b];
  constant += (o[last] / lanes) * stick_stride + o[last] % lanes;
  *walks_stick_to_end = false;
  for (int i = 0; i < rank; ++i) {
    dims[i] = SideDim{false, 0, 0};
    if (size[i] <= 1) continue;
    const int64_t st = v.strides[i];
    if (st == 0) {
      if (is_dst) return TS_ERR_UNSUPPORTED;   // several indices would write one element
      continue;
    }
    if (st < 0) return TS_ERR_UNSUPPORTED;
    int found = -1;
    for (int b = 0; b < v.nb && found < 0; ++b) {
      if (used[b] || v.base[b] <= 1 || st % rm[b]) continue;
      if (o[b] + (size[i] - 1) * (st / rm[b]) < v.base[b]) found = b;
    }
    if (found < 0) return TS_ERR_UNSUPPORTED;
    used[found] = true;
    const int64_t k = st / rm[found];
    if (found != last) {
      dims[i].step = k * img[found];
      continue;
    }
    const bool to_end = k == 1 && o[last] + size[i] == v.base[last];
    const bool inside = o[last] % lanes + (size[i] - 1) * k < lanes;
    // a destination whose last stick has pad lanes gets them zeroed, which the split form does
    const bool must_pad = is_dst && to_end && v.base[last] % lanes != 0;
    if (inside && !must_pad) {
      dims[i].step = k;                       // stays inside one stick
    } else if (k == 1 && o[last] % lanes == 0) {
      dims[i] = SideDim{true, 1, stick_stride};
      *walks_stick_to_end = to_end;
    } else {
      return TS_ERR_UNSUPPORTED;
    }
  }
  return constant;
}

int run_view(const char* src, char* dst, int eb, const int64_t* size, int rank, const ViewSide& sv,
             const ViewSide& dv, cudaStream_t st) {
  if (rank < 1 || rank > kMaxDims || !size || !sv.base || !dv.base || !sv.strides || !dv.strides)
    return TS_ERR_INVALID;
  if (eb != 1 && eb != 2 && eb != 4 && eb != 8) return TS_ERR_INVALID;
  for (int i = 0; i < rank; ++i) {
    if (size[i] < 0) return TS_ERR_INVALID;
    if (size[i] == 0) return TS_OK;
  }
  if (!src || !dst) return TS_ERR_INVALID;
  const int lanes = kStickBytes / eb;
  SideDim sd[kMaxDims], dd[kMaxDims];
  bool s_end, d_end;
  const int64_t soff = decompose_side(sv, size, rank, lanes, false, sd, &s_end);
  if (soff < 0) return (int)soff;
  const int64_t doff = decompose_side(dv, size, rank, lanes, true, dd, &d_end);
  if (doff < 0) return (int)doff;
  // Iteration dims: a view dim split on either side becomes (stick, lane); the side that is
  // not split walks it with strides (lanes * step, step).
  IterDim it[kMaxDims];
  int nd = 0, nchecks = 0;
  int64_t vlimit[kMaxChecks] = {0, 0};
  int vfill[kMaxChecks] = {0, 0};
  for (int i = 0; i < rank; ++i) {
    if (size[i] <= 1) continue;
    const bool split = sd[i].split || dd[i].split;
    if (!split) {
      if (nd == kMaxDims) return TS_ERR_UNSUPPORTED;
      it[nd++] = IterDim{size[i], sd[i].step, dd[i].step, {0, 0}};
      continue;
    }
    if (nd + 2 > kMaxDims) return TS_ERR_UNSUPPORTED;
    const int64_t sticks = ceil_div(size[i], lanes);
    IterDim hi{sticks, sd[i].split ? sd[i].hi_step : sd[i].step * lanes,
               dd[i].split ? dd[i].hi_step : dd[i].step * lanes, {0, 0}};
    IterDim lo{lanes, sd[i].step, dd[i].step, {0, 0}};
    if (size[i] % lanes) {
      if (nchecks == kMaxChecks) return TS_ERR_UNSUPPORTED;
      hi.vm[nchecks] = lanes;
      lo.vm[nchecks] = 1;
      vlimit[nchecks] = size[i];
      // lanes past the end are pad lanes of the destination image (to be zeroed) only when the
      // destination walks its stick dim here and reaches the end of it; anywhere else they are
      // other elements, or do not exist
      vfill[nchecks] = (dd[i].split && d_end) ? 1 : 0;
      ++nchecks;
    }
    it[nd++] = hi;
    it[nd++] = lo;
  }
  if (dv.base[dv.nb - 1] == 1) {
    // one value per stick in the destination: a lane dim that repeats the value, of which only
    // lane 0 exists, zeroes the other lanes
    if (nd == kMaxDims || nchecks == kMaxChecks) return TS_ERR_UNSUPPORTED;
    IterDim lo{lanes, 0, 1, {0, 0}};
    lo.vm[nchecks] = 1;
    vlimit[nchecks] = 1;
    vfill[nchecks] = 1;
    ++nchecks;
    it[nd++] = lo;
  }
  if (nd == 0) it[nd++] = IterDim{1, 1, 1, {0, 0}};
  return plan_and_launch(it, nd, nchecks, vlimit, vfill, kPerCheck, eb, src + soff * eb, dst + doff * eb, st);
}

// Lowest and one-past-highest element offsets a non-negatively strided host tensor touches.
int64_t host_span_elems(const int64_t* size, const int64_t* strides, int rank) {
  int64_t hi = 0;
  for (int h = 0; h < rank; ++h) {
    if (size[h] == 0) return 0;
    hi += (size[h] - 1) * strides[h];
  }
  return hi + 1;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int ts_relayout_to_sticks(const void* strided, void* sticks, int elem_bytes,
                                     const int64_t* host_size, const int64_t* host_strides, int rank,
                                     const int64_t* device_size, const int64_t* device_strides,
                                     const int32_t* dim_map, int ndev, void* stream) {
  Request rq{(const char*)strided, (char*)sticks, true, elem_bytes, host_size, host_strides, rank,
             device_size, device_strides, dim_map, ndev};
  return run(rq, (cudaStream_t)stream);
}

extern "C" int ts_relayout_from_sticks(const void* sticks, void* strided, int elem_bytes,
                                       const int64_t* host_size, const int64_t* host_strides,
                                       int rank, const int64_t* device_size,
                                       const int64_t* device_strides, const int32_t* dim_map,
                                       int ndev, void* stream) {
  Request rq{(const char*)sticks, (char*)strided, false, elem_bytes, host_size, host_strides, rank,
             device_size, device_strides, dim_map, ndev};
  return run(rq, (cudaStream_t)stream);
}

extern "C" int64_t ts_host_span_bytes(int elem_bytes, const int64_t* host_size,
                                      const int64_t* host_strides, int rank) {
  if (!host_size || !host_strides || rank < 0 || rank > kMaxDims) return TS_ERR_INVALID;
  for (int h = 0; h < rank; ++h)
    if (host_strides[h] < 0 || host_size[h] < 0) return TS_ERR_INVALID;
  return host_span_elems(host_size, host_strides, rank) * elem_bytes;
}

extern "C" int ts_copy_host_to_sticks(const void* host, void* staging, void* sticks, int elem_bytes,
                                      const int64_t* host_size, const int64_t* host_strides,
                                      int rank, const int64_t* device_size,
                                      const int64_t* device_strides, const int32_t* dim_map,
                                      int ndev, void* stream) {
  const int64_t bytes = ts_host_span_bytes(elem_bytes, host_size, host_strides, rank);
  if (bytes < 0) return (int)bytes;
  if (bytes > 0) {
    if (!host || !staging) return TS_ERR_INVALID;
    if (cudaMemcpyAsync(staging, host, (size_t)bytes, cudaMemcpyHostToDevice,
                        (cudaStream_t)stream) != cudaSuccess)
      return TS_ERR_CUDA;
  }
  return ts_relayout_to_sticks(staging, sticks, elem_bytes, host_size, host_strides, rank,
                               device_size, device_strides, dim_map, ndev, stream);
}

extern "C" int ts_copy_sticks_to_host(const void* sticks, void* staging, void* host, int elem_bytes,
                                      const int64_t* host_size, const int64_t* host_strides,
                                      int rank, const int64_t* device_size,
                                      const int64_t* device_strides, const int32_t* dim_map,
                                      int ndev, void* stream) {
  const int64_t bytes = ts_host_span_bytes(elem_bytes, host_size, host_strides, rank);
  if (bytes < 0) return (int)bytes;
  if (bytes == 0) return TS_OK;
  if (!host || !staging) return TS_ERR_INVALID;
  int rc = ts_relayout_from_sticks(sticks, staging, elem_bytes, host_size, host_strides, rank,
                                   device_size, device_strides, dim_map, ndev, stream);
  if (rc != TS_OK) return rc;
  if (cudaMemcpyAsync(host, staging, (size_t)bytes, cudaMemcpyDeviceToHost,
                      (cudaStream_t)stream) != cudaSuccess)
    return TS_ERR_CUDA;
  return TS_OK;
}

// ---- pipelined host <-> device copies ------------------------------------------------------
// The host span is moved in chunks of whole leading-dim slices through two halves of a small
// staging buffer: the PCIe copy of chunk k+1 runs on an internal copy stream while the relayout
// kernel of chunk k runs on the caller's stream, and the staging footprint is two chunks instead of
// the whole span.  One copy stream and four events per device, created on first use.
namespace tsb {
namespace {

constexpr int64_t kChunkBytes = 8ll << 20;
constexpr int64_t kMaxChunkBytes = 128ll << 20;   // a leading slice larger than this is not worth two copies of
constexpr int kMaxDevices = 64;

struct CopyPipe {
  std::mutex mu;
  bool ready = false, failed = false;
  cudaStream_t copy = nullptr;
  cudaEvent_t copied[2] = {nullptr, nullptr}, relaid[2] = {nullptr, nullptr};
  // pinned bounce blocks for pageable host memory, one per staging half, grown on demand
  void* pin[2] = {nullptr, nullptr};
  int64_t pin_bytes = 0;
};

// ---- pageable host memory ---------------------------------------------------------------------
// cudaMemcpyAsync on pageable memory is staged by the driver through one thread's memcpy, about
// 10 GB/s here, and a freshly allocated destination (what `.cpu()` returns) adds its page faults to
// that thread: 2 GB/s.  For chunked copies of pageable tensors the library stages the chunks
// itself instead: a few threads copy between the tensor and a pinned block (the page faults of a
// fresh destination spread over them) while the DMA engine moves the neighbouring chunk.
constexpr int64_t kBounceMinBytes = 4ll << 20;   // smaller copies are not worth the threads
constexpr int64_t kBounceMaxChunk = 32ll << 20;  // largest chunk a pinned block is grown to

bool is_pageable(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;   // unknown: leave it to the driver
  }
  return attr.type == cudaMemoryTypeUnregistered;
}

// Helper threads that live for one copy call (nothing outlives the call, so a later fork() of the
// process finds no thread of the library missing).  copy() splits a span into page-aligned
// slices, one per thread, and returns when all are done.
class HostCopyTeam {
 public:
  explicit HostCopyTeam(int threads) {
    for (int i = 1; i < threads; ++i) {
      try {
        helpers_.emplace_back([this, i] { worker(i); });
      } catch (...) {
        break;   // fewer helpers: the slices just get larger
      }
    }
    n_ = (int)helpers_.size() + 1;
  }
  ~HostCopyTeam() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stop_ = true;
    }
    cv_start_.notify_all();
    for (auto& t : helpers_) t.join();
  }
  void copy(void* dst, const void* src, size_t bytes) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      dst_ = (char*)dst;
      src_ = (const char*)src;
      bytes_ = bytes;
      slice_ = ((bytes / n_ + 4095) / 4096 + 1) * 4096;
      pending_ = n_ - 1;
      ++generation_;
    }
    cv_start_.notify_all();
    copy_slice(0);
    std::unique_lock<std::mutex> lock(mu_);
    cv_done_.wait(lock, [this] { return pending_ == 0; });
  }

 private:
  void copy_slice(int id) {
    const size_t lo = std::min(bytes_, (size_t)id * slice_), hi = std::min(bytes_, lo + slice_);
    if (hi > lo) std::memcpy(dst_ + lo, src_ + lo, hi - lo);
  }
  void worker(int id) {
    uint64_t seen = 0;
    std::unique_lock<std::mutex> lock(mu_);
    for (;;) {
      cv_start_.wait(lock, [&] { return stop_ || generation_ != seen; });
      if (stop_) return;
      seen = generation_;
      lock.unlock();
      copy_slice(id);
      lock.lock();
      if (--pending_ == 0) cv_done_.notify_one();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_start_, cv_done_;
  std::vector<std::thread> helpers_;
  char* dst_ = nullptr;
  const char* src_ = nullptr;
  size_t bytes_ = 0, slice_ = 0;
  uint64_t generation_ = 0;
  int pending_ = 0, n_ = 1;
  bool stop_ = false;
};

// A destination that was only just allocated (the result of `.cpu()`) takes a page fault for
// every 4 KiB the threads write.  Asking for transparent huge pages over its 2 MiB-aligned
// interior turns those into one fault per 2 MiB where the system allows it ("madvise" or
// "always" mode): 5.3 -> 9.8 GB/s for a fresh 128 MiB destination, no change for one that is
// already backed by pages (measured in one process).  For memory that is not anonymous, or where
// the system says "never", the call fails or does nothing.
void advise_huge_pages(void* p, int64_t bytes) {
#ifdef MADV_HUGEPAGE
#ifdef TSB_TUNING
  const char* knob = getenv("TS_COPY_HUGEPAGE");   // experiment: 0 = never
  if (knob && knob[0] == '0') return;
#endif
  const uintptr_t two_mib = (uintptr_t)2 << 20;
  const uintptr_t lo = ((uintptr_t)p + two_mib - 1) & ~(two_mib - 1), hi = ((uintptr_t)p + (uintptr_t)bytes) & ~(two_mib - 1);
  if (hi > lo) (void)madvise((void*)lo, hi - lo, MADV_HUGEPAGE);
#else
  (void)p;
  (void)bytes;
#endif
}

int bounce_threads() {
  const unsigned hw = std::thread::hardware_concurrency();
  return (int)std::min(8u, std::max(2u, hw / 4));
}

// Makes both pinned blocks at least `bytes` large.  Called with the pipe's mutex held and no DMA
// of an earlier call still using the blocks (the callers wait for the `copied` events first).
bool grow_bounce(CopyPipe* pipe, int64_t bytes) {
  if (pipe->pin_bytes >= bytes) return true;
  for (int i = 0; i < 2; ++i) {
    if (pipe->pin[i]) cudaFreeHost(pipe->pin[i]);
    pipe->pin[i] = nullptr;
  }
  pipe->pin_bytes = 0;
  for (int i = 0; i < 2; ++i) {
    if (cudaHostAlloc(&pipe->pin[i], (size_t)bytes, cudaHostAllocDefault) != cudaSuccess) {
      cudaGetLastError();
      for (int j = 0; j < 2; ++j) {
        if (pipe->pin[j]) cudaFreeHost(pipe->pin[j]);
        pipe->pin[j] = nullptr;
      }
      return false;
    }
  }
  pipe->pin_bytes = bytes;
  return true;
}

// Whether this chunked copy goes through the pinned blocks, which are then ready for it.
bool use_bounce(CopyPipe* pipe, const void* host, int64_t bytes, int64_t chunk_span) {
  if (bytes < kBounceMinBytes || chunk_span > kBounceMaxChunk || !is_pageable(host)) return false;
  // the blocks may still be the source or target of an earlier call's last DMAs
  if (cudaEventSynchronize(pipe->copied[0]) != cudaSuccess || cudaEventSynchronize(pipe->copied[1]) != cudaSuccess)
    return false;
  return grow_bounce(pipe, (chunk_span + 4095) & ~(int64_t)4095);
}
CopyPipe g_pipes[kMaxDevices];

CopyPipe* pipe_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  CopyPipe* p = &g_pipes[dev];
  std::lock_guard<std::mutex> lock(p->mu);
  if (!p->ready && !p->failed) {
    bool ok = cudaStreamCreateWithFlags(&p->copy, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < 2 && ok; ++i)
      ok = cudaEventCreateWithFlags(&p->copied[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p->relaid[i], cudaEventDisableTiming) == cudaSuccess;
    p->ready = ok;
    p->failed = !ok;
  }
  return p->ready ? p : nullptr;
}

struct ChunkPlan {
  bool chunked = false;
  int dev_dim = -1;           // the device dim that walks host dim 0
  int64_t rows_per_chunk = 0, row_bytes = 0, rest_bytes = 0;
};

// Whether (and how) a copy can be cut along host dim 0: slices must be disjoint, ascending spans of
// host memory, and host dim 0 must be one whole device dim (not the stick dim).
ChunkPlan plan_chunks(int eb, const int64_t* hsize, const int64_t* hstr, int rank, const int32_t* dim_map,
                      int ndev, int64_t staging_bytes) {
  ChunkPlan c;
  if (rank < 2 || hsize[0] < 2) return c;
  int count = 0;
  for (int d = 0; d < ndev; ++d)
    if (dim_map[d] == 0) { c.dev_dim = d; ++count; }
  if (count != 1) return c;
  const int64_t rest = host_span_elems(hsize + 1, hstr + 1, rank - 1);
  if (rest <= 0 || hstr[0] < rest) return c;
  c.row_bytes = hstr[0] * eb;
  c.rest_bytes = rest * eb;
  // a chunk is about kChunkBytes, at least one leading slice, and fits half the staging block
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  const int64_t target = std::min(half, std::max(kChunkBytes, c.rest_bytes));
  if (target < c.rest_bytes) return c;
  c.rows_per_chunk = 1 + (target - c.rest_bytes) / c.row_bytes;
  c.chunked = c.rows_per_chunk < hsize[0];
  return c;
}

}  // namespace
}  // namespace tsb

extern "C" int64_t ts_copy_staging_bytes(int elem_bytes, const int64_t* host_size,
                                         const int64_t* host_strides, int rank) {
  const int64_t span = ts_host_span_bytes(elem_bytes, host_size, host_strides, rank);
  if (span < 0) return span;
  int64_t chunk = kChunkBytes;
  if (rank >= 2 && host_size[0] >= 2) {   // room for at least one leading slice per half, within reason
    const int64_t rest = host_span_elems(host_size + 1, host_strides + 1, rank - 1) * elem_bytes;
    if (rest > chunk && rest <= kMaxChunkBytes) chunk = (rest + 255) & ~(int64_t)255;
  }
  return std::min<int64_t>((span + 255) & ~(int64_t)255, 2 * chunk);
}

extern "C" int ts_host_copy_selftest(void* dst, const void* src, int64_t bytes, int threads) {
  if (bytes < 0 || threads < 1 || threads > 64 || (bytes > 0 && (!dst || !src))) return TS_ERR_INVALID;
  tsb::HostCopyTeam team(threads);
  for (int rep = 0; rep < 2; ++rep)   // twice: a team serves every chunk of a call
    team.copy(dst, src, (size_t)bytes);
  return TS_OK;
}

extern "C" int ts_copy_host_to_sticks_pipelined(const void* host, void* staging, int64_t staging_bytes,
                                                void* sticks, int elem_bytes, const int64_t* host_size,
                                                const int64_t* host_strides, int rank,
                                                const int64_t* device_size, const int64_t* device_strides,
                                                const int32_t* dim_map, int ndev, void* stream) {
  const int64_t bytes = ts_host_span_bytes(elem_bytes, host_size, host_strides, rank);
  if (bytes < 0) return (int)bytes;
  if (rank < 1 || rank > kMaxDims || ndev < 1 || ndev > kMaxDims || !device_size || !device_strides || !dim_map)
    return TS_ERR_INVALID;
  if (bytes > 0 && (!host || !staging || !sticks)) return TS_ERR_INVALID;
  const ChunkPlan c = plan_chunks(elem_bytes, host_size, host_strides, rank, dim_map, ndev, staging_bytes);
  CopyPipe* pipe = c.chunked ? pipe_for_current_device() : nullptr;
  if (!pipe) {
    if (staging_bytes < bytes) return TS_ERR_TOO_LARGE;
    return ts_copy_host_to_sticks(host, staging, sticks, elem_bytes, host_size, host_strides, rank,
                                  device_size, device_strides, dim_map, ndev, stream);
  }
  cudaStream_t st = (cudaStream_t)stream;
  std::lock_guard<std::mutex> lock(pipe->mu);
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  int64_t hs[kMaxDims], ds[kMaxDims];
  for (int i = 0; i < rank; ++i) hs[i] = host_size[i];
  for (int i = 0; i < ndev; ++i) ds[i] = device_size[i];
  // the copy stream may not touch the staging block before work already queued on `stream` is done with it
  if (cudaEventRecord(pipe->relaid[0], st) != cudaSuccess ||
      cudaStreamWaitEvent(pipe->copy, pipe->relaid[0], 0) != cudaSuccess) return TS_ERR_CUDA;
  const int64_t chunk_span = (std::min(c.rows_per_chunk, host_size[0]) - 1) * c.row_bytes + c.rest_bytes;
  const bool bounce = use_bounce(pipe, host, bytes, chunk_span);
  HostCopyTeam team(bounce ? bounce_threads() : 1);
  int k = 0;
  for (int64_t r0 = 0; r0 < host_size[0]; r0 += c.rows_per_chunk, ++k) {
    const int slot = k & 1;
    const int64_t rows = std::min(c.rows_per_chunk, host_size[0] - r0);
    const int64_t span = (rows - 1) * c.row_bytes + c.rest_bytes;
    char* stage = (char*)staging + slot * half;
    const char* from = (const char*)host + r0 * c.row_bytes;
    if (bounce) {
      // the DMA that last read this pinned block (chunk k - 2) must be done before it is refilled;
      // the threads fill it while the DMA of chunk k - 1 runs
      if (k >= 2 && cudaEventSynchronize(pipe->copied[slot]) != cudaSuccess) return TS_ERR_CUDA;
      team.copy(pipe->pin[slot], from, (size_t)span);
      from = (const char*)pipe->pin[slot];
    }
    if (k >= 2 && cudaStreamWaitEvent(pipe->copy, pipe->relaid[slot], 0) != cudaSuccess) return TS_ERR_CUDA;
    if (cudaMemcpyAsync(stage, from, (size_t)span, cudaMemcpyHostToDevice,
                        pipe->copy) != cudaSuccess ||
        cudaEventRecord(pipe->copied[slot], pipe->copy) != cudaSuccess ||
        cudaStreamWaitEvent(st, pipe->copied[slot], 0) != cudaSuccess)
      return TS_ERR_CUDA;
    hs[0] = rows;
    ds[c.dev_dim] = rows;
    const int rc = ts_relayout_to_sticks(stage, (char*)sticks + r0 * device_strides[c.dev_dim] * elem_bytes,
                                         elem_bytes, hs, host_strides, rank, ds, device_strides, dim_map, ndev,
                                         stream);
    if (rc != TS_OK) return rc;
    if (cudaEventRecord(pipe->relaid[slot], st) != cudaSuccess) return TS_ERR_CUDA;
  }
  return TS_OK;
}

extern "C" int ts_copy_sticks_to_host_pipelined(const void* sticks, void* staging, int64_t staging_bytes,
                                                void* host, int elem_bytes, const int64_t* host_size,
                                                const int64_t* host_strides, int rank,
                                                const int64_t* device_size, const int64_t* device_strides,
                                                const int32_t* dim_map, int ndev, void* stream) {
  const int64_t bytes = ts_host_span_bytes(elem_bytes, host_size, host_strides, rank);
  if (bytes < 0) return (int)bytes;
  if (bytes == 0) return TS_OK;
  if (rank < 1 || rank > kMaxDims || ndev < 1 || ndev > kMaxDims || !device_size || !device_strides || !dim_map)
    return TS_ERR_INVALID;
  if (!host || !staging || !sticks) return TS_ERR_INVALID;
  ChunkPlan c = plan_chunks(elem_bytes, host_size, host_strides, rank, dim_map, ndev, staging_bytes);
  // a host tensor with gaps keeps its gap bytes only on the single-shot path (whose caller
  // preloads the staging image with them)
  int64_t dense = elem_bytes;
  for (int i = 0; i < rank; ++i) dense *= host_size[i];
  if (dense != bytes) c.chunked = false;
  CopyPipe* pipe = c.chunked ? pipe_for_current_device() : nullptr;
  if (!pipe) {
    if (staging_bytes < bytes) return TS_ERR_TOO_LARGE;
    return ts_copy_sticks_to_host(sticks, staging, host, elem_bytes, host_size, host_strides, rank, device_size,
                                  device_strides, dim_map, ndev, stream);
  }
  cudaStream_t st = (cudaStream_t)stream;
  std::lock_guard<std::mutex> lock(pipe->mu);
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  int64_t hs[kMaxDims], ds[kMaxDims];
  for (int i = 0; i < rank; ++i) hs[i] = host_size[i];
  for (int i = 0; i < ndev; ++i) ds[i] = device_size[i];
  const int64_t chunk_span = (std::min(c.rows_per_chunk, host_size[0]) - 1) * c.row_bytes + c.rest_bytes;
  const bool bounce = use_bounce(pipe, host, bytes, chunk_span);
  HostCopyTeam team(bounce ? bounce_threads() : 1);
  if (bounce) advise_huge_pages(host, bytes);
  char* landed_to = nullptr;      // with the bounce: where the chunk before this one goes, and its size
  int64_t landed_span = 0;
  int k = 0;
  for (int64_t r0 = 0; r0 < host_size[0]; r0 += c.rows_per_chunk, ++k) {
    const int slot = k & 1;
    const int64_t rows = std::min(c.rows_per_chunk, host_size[0] - r0);
    const int64_t span = (rows - 1) * c.row_bytes + c.rest_bytes;
    char* stage = (char*)staging + slot * half;
    // the slot's previous contents must have left for the host
    if (k >= 2 && cudaStreamWaitEvent(st, pipe->copied[slot], 0) != cudaSuccess) return TS_ERR_CUDA;
    hs[0] = rows;
    ds[c.dev_dim] = rows;
    const int rc = ts_relayout_from_sticks((const char*)sticks + r0 * device_strides[c.dev_dim] * elem_bytes, stage,
                                           elem_bytes, hs, host_strides, rank, ds, device_strides, dim_map, ndev,
                                           stream);
    if (rc != TS_OK) return rc;
    char* to = (char*)host + r0 * c.row_bytes;
    if (cudaEventRecord(pipe->relaid[slot], st) != cudaSuccess ||
        cudaStreamWaitEvent(pipe->copy, pipe->relaid[slot], 0) != cudaSuccess ||
        cudaMemcpyAsync(bounce ? (char*)pipe->pin[slot] : to, stage, (size_t)span, cudaMemcpyDeviceToHost,
                        pipe->copy) != cudaSuccess ||
        cudaEventRecord(pipe->copied[slot], pipe->copy) != cudaSuccess)
      return TS_ERR_CUDA;
    if (bounce) {
      // while this chunk's DMA runs, the threads move the one before it from its pinned block to
      // the tensor (that block is not written again before the next iteration's DMA)
      if (landed_to) {
        if (cudaEventSynchronize(pipe->copied[slot ^ 1]) != cudaSuccess) return TS_ERR_CUDA;
        team.copy(landed_to, pipe->pin[slot ^ 1], (size_t)landed_span);
      }
      landed_to = to;
      landed_span = span;
    }
  }
  if (bounce && landed_to) {
    const int last = (k - 1) & 1;
    if (cudaEventSynchronize(pipe->copied[last]) != cudaSuccess) return TS_ERR_CUDA;
    team.copy(landed_to, pipe->pin[last], (size_t)landed_span);
  }
  // synchronising `stream` must cover the copies
  for (int slot = 0; slot < 2 && slot < k; ++slot)
    if (cudaStreamWaitEvent(st, pipe->copied[slot], 0) != cudaSuccess) return TS_ERR_CUDA;
  return TS_OK;
}

extern "C" int ts_layout_init(const int64_t* host_size, int rank, int elem_bytes,
                              const int32_t* dim_order, int64_t* device_size,
                              int64_t* device_strides, int32_t* dim_map) {
  if (!host_size || !device_size || !device_strides || !dim_map) return TS_ERR_INVALID;
  if (rank < 1 || rank + 1 > kMaxDims) return TS_ERR_INVALID;
  if (elem_bytes < 1 || kStickBytes % elem_bytes) return TS_ERR_INVALID;
  const int ndev = rank + 1;
  const int64_t elems = kStickBytes / elem_bytes;
  auto order = [&](int i) { return dim_order ? dim_order[i] : i; };
  for (int i = 0; i < rank; ++i)
    if (order(i) < 0 || order(i) >= rank) return TS_ERR_INVALID;
  const int stick_dim = order(rank - 1);
  dim_map[0] = stick_dim;
  dim_map[ndev - 1] = stick_dim;
  device_size[0] = (host_size[stick_dim] + elems - 1) / elems;
  device_size[ndev - 1] = elems;
  for (int i = 1; i < ndev - 1; ++i) {
    dim_map[i] = order(i - 1);
    device_size[i] = host_size[order(i - 1)];
  }
  int64_t cur = elems;
  device_strides[ndev - 1] = 1;
  for (int i = ndev - 2; i >= 0; --i) {
    device_strides[i] = cur;
    cur *= device_size[i];
  }
  return ndev;
}

extern "C" int ts_transpose_tiles(const void* src_sticks, const int64_t* src_base, int src_base_rank,
                                  const int64_t* src_strides, int64_t src_offset, void* dst_sticks,
                                  const int64_t* dst_base, int dst_base_rank, const int64_t* dst_strides,
                                  int64_t dst_offset, const int64_t* size, int rank, int elem_bytes,
                                  void* stream) {
  const ViewSide sv{src_base, src_base_rank, src_strides, src_offset};
  const ViewSide dv{dst_base, dst_base_rank, dst_strides, dst_offset};
  return run_view((const char*)src_sticks, (char*)dst_sticks, elem_bytes, size, rank, sv, dv,
                  (cudaStream_t)stream);
}
