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

#include "common.cuh"

namespace tsb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnitsPerThread = 4;
constexpr int kTileUnits = kThreads * kUnitsPerThread;  // 1024
constexpr int kMaxChecks = 2;

struct CopyPlan {
  int nd;                        // iteration dims, outermost first
  uint32_t size[kMaxDims];       // extent per dim (last dim of copy_tiles: in units)
  int64_t sbytes[kMaxDims];      // source stride per dim, bytes
  int64_t dbytes[kMaxDims];      // destination stride per dim, bytes
  uint32_t tile[kMaxDims];       // tile extent per dim (1 = not tiled)
  FastDiv ntiles[kMaxDims];      // tiles per dim
  // Padding: index is inside the host tensor iff, for every check c,
  // sum_d idx[d] * vmul[c][d] < vlimit[c].
  int nchecks;
  int64_t vmul[kMaxChecks][kMaxDims];
  int64_t vlimit[kMaxChecks];
  // copy_tiles: tile = T0 (dim nd-1) x T1 (dim tx) x T2 (dim ty), powers of two.
  int tx, ty, log_t0, log_t1;
  uint32_t t2;
  // transpose_tiles: dim `ta` is unit-stride in the source, `tb` in the destination.
  int ta, tb;
};

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

__device__ __forceinline__ void decode_tile(const CopyPlan& p, uint32_t tile_id, uint32_t* origin) {
  uint32_t rem = tile_id;
#pragma unroll
  for (int d = kMaxDims - 1; d >= 0; --d) {
    if (d < p.nd) {
      uint32_t q, r;
      p.ntiles[d].divmod(rem, q, r);
      origin[d] = r * p.tile[d];
      rem = q;
    }
  }
}

// ---------------------------------------------------------------------------
template <int UNIT, bool TO_DEVICE>
__global__ void __launch_bounds__(kThreads)
copy_tiles(const __grid_constant__ CopyPlan p, const char* __restrict__ src, char* __restrict__ dst) {
  using T = typename UnitType<UNIT>::T;
  uint32_t origin[kMaxDims];
  decode_tile(p, blockIdx.x, origin);
  int64_t soff = 0, doff = 0, v[kMaxChecks] = {0, 0};
#pragma unroll
  for (int d = 0; d < kMaxDims; ++d) {
    if (d < p.nd) {
      soff += (int64_t)origin[d] * p.sbytes[d];
      doff += (int64_t)origin[d] * p.dbytes[d];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c)
        if (c < p.nchecks) v[c] += (int64_t)origin[d] * p.vmul[c][d];
    }
  }
  const int d0 = p.nd - 1, dx = p.tx, dy = p.ty;
  const uint32_t m0 = (1u << p.log_t0) - 1, m1 = (1u << p.log_t1) - 1;
  T val[kUnitsPerThread];
  int64_t dpos[kUnitsPerThread];
  bool live[kUnitsPerThread];
#pragma unroll
  for (int k = 0; k < kUnitsPerThread; ++k) {
    const uint32_t t = threadIdx.x + k * kThreads;
    const uint32_t i0 = t & m0, i1 = (t >> p.log_t0) & m1, i2 = t >> (p.log_t0 + p.log_t1);
    bool inb = origin[d0] + i0 < p.size[d0];
    int64_t so = soff + (int64_t)i0 * p.sbytes[d0], dof = doff + (int64_t)i0 * p.dbytes[d0];
    int64_t vv[kMaxChecks];
#pragma unroll
    for (int c = 0; c < kMaxChecks; ++c) vv[c] = v[c] + (int64_t)i0 * p.vmul[c][d0];
    if (dx >= 0) {
      inb = inb && (origin[dx] + i1 < p.size[dx]);
      so += (int64_t)i1 * p.sbytes[dx];
      dof += (int64_t)i1 * p.dbytes[dx];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c) vv[c] += (int64_t)i1 * p.vmul[c][dx];
    } else {
      inb = inb && (i1 == 0);
    }
    if (dy >= 0) {
      inb = inb && (i2 < p.t2) && (origin[dy] + i2 < p.size[dy]);
      so += (int64_t)i2 * p.sbytes[dy];
      dof += (int64_t)i2 * p.dbytes[dy];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c) vv[c] += (int64_t)i2 * p.vmul[c][dy];
    } else {
      inb = inb && (i2 == 0);
    }
    bool valid = true;
#pragma unroll
    for (int c = 0; c < kMaxChecks; ++c)
      if (c < p.nchecks) valid = valid && (vv[c] < p.vlimit[c]);
    val[k] = zero_of<T>();
    if (inb && valid) val[k] = *reinterpret_cast<const T*>(src + so);
    live[k] = inb && (TO_DEVICE || valid);
    dpos[k] = dof;
  }
#pragma unroll
  for (int k = 0; k < kUnitsPerThread; ++k)
    if (live[k]) *reinterpret_cast<T*>(dst + dpos[k]) = val[k];
}

// ---------------------------------------------------------------------------
// 64x64 tile of 2-byte elements.  smem holds the tile as [row = tb index][col =
// ta index], 32-bit words, pitch 33 words so that both phases are conflict free.
constexpr int kTT = 64;
constexpr int kPitchWords = 33;

// Number of leading elements (0..8), along a dim whose check multipliers are
// `mul`, that satisfy every check, given the check sums at the first element.
__device__ __forceinline__ int valid_run(const CopyPlan& p, const int64_t* vsum, int dim) {
  int n = 8;
#pragma unroll
  for (int c = 0; c < kMaxChecks; ++c) {
    if (c < p.nchecks) {
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

template <bool TO_DEVICE, bool VEC_IN, bool VEC_OUT>
__global__ void __launch_bounds__(kThreads)
transpose_tiles(const __grid_constant__ CopyPlan p, const char* __restrict__ src,
                char* __restrict__ dst) {
  __shared__ uint32_t tile[kTT * kPitchWords];
  uint32_t origin[kMaxDims];
  decode_tile(p, blockIdx.x, origin);
  int64_t soff = 0, doff = 0, v[kMaxChecks] = {0, 0};
#pragma unroll
  for (int d = 0; d < kMaxDims; ++d) {
    if (d < p.nd) {
      soff += (int64_t)origin[d] * p.sbytes[d];
      doff += (int64_t)origin[d] * p.dbytes[d];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c)
        if (c < p.nchecks) v[c] += (int64_t)origin[d] * p.vmul[c][d];
    }
  }
  const int da = p.ta, db = p.tb;
  const int rem_a = (int)min((uint32_t)kTT, p.size[da] - origin[da]);
  const int rem_b = (int)min((uint32_t)kTT, p.size[db] - origin[db]);

  // Phase 1: rows along tb, 16-byte vectors along ta.
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int row = (threadIdx.x >> 3) + k * 32;
    const int vec = threadIdx.x & 7;
    uint32_t w[4] = {0, 0, 0, 0};
    int na = rem_a - vec * 8;
    na = na < 0 ? 0 : (na > 8 ? 8 : na);
    if (row >= rem_b) na = 0;
    if (TO_DEVICE && na > 0) {
      int64_t vs[kMaxChecks];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c)
        vs[c] = v[c] + (int64_t)row * p.vmul[c][db] + (int64_t)(vec * 8) * p.vmul[c][da];
      na = min(na, valid_run(p, vs, da));
    }
    const char* sp = src + soff + (int64_t)row * p.sbytes[db] + vec * 16;
    if (VEC_IN && na == 8) {
      const uint4 q = ld_stream_v4(sp);
      w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < na) {
          const uint32_t e = *reinterpret_cast<const uint16_t*>(sp + 2 * j);
          w[j >> 1] |= e << ((j & 1) * 16);
        }
      }
    }
    uint32_t* tp = &tile[row * kPitchWords + vec * 4];
    tp[0] = w[0]; tp[1] = w[1]; tp[2] = w[2]; tp[3] = w[3];
  }
  __syncthreads();

  // Phase 2: output rows along ta (two per thread), 8 consecutive tb per thread.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pcol = 8 * (warp & 3) + (lane & 7);   // word column: ta = 2*pcol, 2*pcol+1
  const int grp = 4 * (warp >> 2) + (lane >> 3);  // tb = 8*grp .. 8*grp+7
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = tile[(8 * grp + j) * kPitchWords + pcol];
  int nb = rem_b - grp * 8;
  nb = nb < 0 ? 0 : (nb > 8 ? 8 : nb);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int a = 2 * pcol + half;
    if (a >= rem_a) continue;
    int n = nb;
    if (!TO_DEVICE && n > 0) {
      int64_t vs[kMaxChecks];
#pragma unroll
      for (int c = 0; c < kMaxChecks; ++c)
        vs[c] = v[c] + (int64_t)a * p.vmul[c][da] + (int64_t)(grp * 8) * p.vmul[c][db];
      n = min(n, valid_run(p, vs, db));
    }
    const uint32_t sel = half ? 0x7632u : 0x5410u;
    uint4 q;
    q.x = __byte_perm(w[0], w[1], sel);
    q.y = __byte_perm(w[2], w[3], sel);
    q.z = __byte_perm(w[4], w[5], sel);
    q.w = __byte_perm(w[6], w[7], sel);
    char* dp = dst + doff + (int64_t)a * p.dbytes[da] + grp * 16;
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

template <bool TO_DEVICE>
int launch_copy(const CopyPlan& plan, int unit, uint32_t blocks, const char* src, char* dst,
                cudaStream_t st) {
  switch (unit) {
    case 16: copy_tiles<16, TO_DEVICE><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 8: copy_tiles<8, TO_DEVICE><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 4: copy_tiles<4, TO_DEVICE><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    case 2: copy_tiles<2, TO_DEVICE><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
    default: copy_tiles<1, TO_DEVICE><<<blocks, kThreads, 0, st>>>(plan, src, dst); break;
  }
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

template <bool TO_DEVICE>
int launch_transpose(const CopyPlan& plan, bool vin, bool vout, uint32_t blocks, const char* src,
                     char* dst, cudaStream_t st) {
  if (vin && vout) transpose_tiles<TO_DEVICE, true, true><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else if (vin) transpose_tiles<TO_DEVICE, true, false><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else if (vout) transpose_tiles<TO_DEVICE, false, true><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  else transpose_tiles<TO_DEVICE, false, false><<<blocks, kThreads, 0, st>>>(plan, src, dst);
  TSB_CHECK_LAUNCH();
  return TS_OK;
}

int run(const Request& rq, cudaStream_t st) {
  if (!rq.host_size || !rq.host_strides || !rq.dev_size || !rq.dev_strides || !rq.dim_map)
    return TS_ERR_INVALID;
  if (rq.rank < 1 || rq.rank > kMaxDims || rq.ndev < 1 || rq.ndev > kMaxDims) return TS_ERR_INVALID;
  if (rq.elem_bytes != 1 && rq.elem_bytes != 2 && rq.elem_bytes != 4) return TS_ERR_INVALID;
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
  // Drop size-1 dims, then merge neighbours that are contiguous on both sides.
  int nd = 0;
  for (int d = 0; d < rq.ndev; ++d)
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
  for (int c = 0; c < kMaxChecks; ++c) plan.vlimit[c] = vlimit[c];

  int ua = -1, ub = -1;  // unit-stride dims of source / destination
  for (int d = 0; d < nd; ++d) {
    if (it[d].s == 1 && ua < 0) ua = d;
    if (it[d].d == 1 && ub < 0) ub = d;
  }
  const uintptr_t sbase = (uintptr_t)rq.src, dbase = (uintptr_t)rq.dst;

  if (eb == 2 && ua >= 0 && ub >= 0 && ua != ub && it[ua].size >= 16 && it[ub].size >= 16) {
    // ---- transpose path
    plan.nd = nd;
    bool vin = sbase % 16 == 0, vout = dbase % 16 == 0;
    uint64_t ntiles = 1;
    for (int d = 0; d < nd; ++d) {
      plan.size[d] = (uint32_t)it[d].size;
      plan.sbytes[d] = it[d].s * eb;
      plan.dbytes[d] = it[d].d * eb;
      plan.tile[d] = (d == ua || d == ub) ? kTT : 1;
      const uint32_t nt = (uint32_t)ceil_div(it[d].size, plan.tile[d]);
      plan.ntiles[d].init(nt);
      ntiles *= nt;
      for (int c = 0; c < kMaxChecks; ++c) plan.vmul[c][d] = it[d].vm[c];
      if (d != ua && plan.sbytes[d] % 16) vin = false;
      if (d != ub && plan.dbytes[d] % 16) vout = false;
    }
    if (ntiles >= (1ull << 31)) return TS_ERR_TOO_LARGE;
    plan.ta = ua;
    plan.tb = ub;
    return rq.to_device ? launch_transpose<true>(plan, vin, vout, (uint32_t)ntiles, rq.src, rq.dst, st)
                        : launch_transpose<false>(plan, vin, vout, (uint32_t)ntiles, rq.src, rq.dst, st);
  }

  // ---- copy path.  Needs an innermost dim with unit stride on both sides; a
  // dummy one of extent 1 is appended when the tensor has none.
  if (!(it[nd - 1].s == 1 && it[nd - 1].d == 1)) {
    if (nd == kMaxDims) return TS_ERR_UNSUPPORTED;
    it[nd] = IterDim{1, 1, 1, {0, 0}};
    ++nd;
  }
  // Widest unit (bytes) dividing every address, the inner extent and the limits.
  int unit = 16;
  auto fits = [&](int u) {
    if (u < eb) return false;
    if (u == eb) return true;
    const int ue = u / eb;
    if (sbase % u || dbase % u) return false;
    if (it[nd - 1].size % ue) return false;
    for (int d = 0; d < nd - 1; ++d)
      if ((it[d].s * eb) % u || (it[d].d * eb) % u) return false;
    for (int c = 0; c < nchecks; ++c)
      if (it[nd - 1].vm[c] != 0 && vlimit[c] % ue) return false;
    return true;
  };
  while (!fits(unit)) unit >>= 1;
  const int ue = unit / eb;
  plan.nd = nd;
  for (int d = 0; d < nd; ++d) {
    const bool last = d == nd - 1;
    plan.size[d] = (uint32_t)(last ? it[d].size / ue : it[d].size);
    plan.sbytes[d] = last ? unit : it[d].s * eb;
    plan.dbytes[d] = last ? unit : it[d].d * eb;
    for (int c = 0; c < kMaxChecks; ++c) plan.vmul[c][d] = it[d].vm[c] * (last ? ue : 1);
    plan.tile[d] = 1;
  }
  // Tile: inner run first, then the dims next-most contiguous in source and in destination.
  const uint32_t t0 = std::min<uint32_t>(pow2_ceil(plan.size[nd - 1]), kTileUnits);
  uint32_t rest = kTileUnits / t0;
  int tx = -1, ty = -1;
  for (int d = 0; d < nd - 1; ++d) {
    if (tx < 0 || llabs(plan.sbytes[d]) < llabs(plan.sbytes[tx])) tx = d;
    if (ty < 0 || llabs(plan.dbytes[d]) < llabs(plan.dbytes[ty])) ty = d;
  }
  uint32_t t1 = 1, t2 = 1;
  if (tx >= 0 && rest > 1) {
    if (tx == ty) {
      t1 = std::min<uint32_t>(rest, pow2_ceil(plan.size[tx]));
      ty = -1;
    } else {
      const uint32_t want = 1u << ((log2_floor(rest) + 1) / 2);
      t1 = std::min<uint32_t>(want, pow2_ceil(plan.size[tx]));
      t2 = std::min<uint32_t>(rest / t1, pow2_ceil(plan.size[ty]));
      // hand unused budget back to the source-side dim
      t1 = std::min<uint32_t>(rest / t2, pow2_ceil(plan.size[tx]));
    }
  } else {
    tx = ty = -1;
  }
  plan.tile[nd - 1] = t0;
  if (tx >= 0) plan.tile[tx] = t1;
  if (ty >= 0) plan.tile[ty] = t2;
  plan.tx = tx;
  plan.ty = ty;
  plan.log_t0 = log2_floor(t0);
  plan.log_t1 = log2_floor(t1);
  plan.t2 = t2;
  uint64_t ntiles = 1;
  for (int d = 0; d < nd; ++d) {
    const uint32_t nt = (uint32_t)ceil_div(plan.size[d], plan.tile[d]);
    plan.ntiles[d].init(nt);
    ntiles *= nt;
  }
  if (ntiles >= (1ull << 31)) return TS_ERR_TOO_LARGE;
  return rq.to_device ? launch_copy<true>(plan, unit, (uint32_t)ntiles, rq.src, rq.dst, st)
                      : launch_copy<false>(plan, unit, (uint32_t)ntiles, rq.src, rq.dst, st);
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
