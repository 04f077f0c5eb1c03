// Backward on the 5th-generation tensor cores: two kernels after a small
// pre-pass, no atomics (every gradient tile has exactly one writer).
//
//   delta[b,h,i] = sum_d O*dO - dLSE                      (bwd_delta_vec_kernel)
//   dQ  kernel: one CTA per 128-row query tile (two 64-row halves as in the
//               forward), walks the union of the halves' CSR rows:
//                 S = Q K^T, dP = dO V^T, dS = exp2(S c - lse) * (dP - delta),
//                 dQ += dS K
//   dKdV kernel: one CTA per pair of adjacent kv blocks of one kv head, walks, for
//               every q head of the group, the union of the two CSC columns:
//                 S^T = K Q^T, dP^T = V dO^T, P^T, dS^T,
//                 dV += P^T dO, dK += dS^T Q
// All products are tcgen05.mma with fp32 accumulators in TMEM; the transposed
// formulation of the dK/dV kernel puts the kv rows on the TMEM lanes, so P^T and
// dS^T are written back by tcgen05.st and consumed as TMEM A operands while Q and
// dO serve as MN-major B operands straight from their TMA tiles.  S/dP are double
// buffered in TMEM (512 columns, one CTA per SM) so the MMAs of step e+1 overlap
// the exponentials of step e.  Element-wise warps own a TMEM lane quadrant and a slice
// of the columns (16 warps x 16 columns in both kernels);
// one TMA producer warp; two MMA issuer warps, because a tcgen05.mma costs its issuing
// thread about as long as a 128x64x16 product takes on the tensor pipe.  The issuers
// split the products along the data paths, so that a product overwriting columns an
// earlier product still reads always follows it in one thread's issue order (the tensor
// pipe executes one thread's products in order) and never waits for a completion.
// Math: dkernel/ops/sparse_attn_bwd.py:86-170
// (dK/dV), :329-419 (dQ), :73-80 (delta); P and dS are rounded to the input
// type before the second-stage products, like the reference (:144,:166,:413).
#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kBS = 64;
constexpr int kDqEwWarps = 16;        // dQ kernel: 16 element-wise warps, producer, two issuers
constexpr int kBwdThreads = 32 * (kDqEwWarps + 3);
constexpr int kWarpProducer = kDqEwWarps, kWarpIssueA = kDqEwWarps + 1, kWarpIssueB = kDqEwWarps + 2;
constexpr int kDkdvEwWarps = 16;      // dK/dV kernel: 16 element-wise warps, producer, two issuers
constexpr int kDkdvThreads = 32 * (kDkdvEwWarps + 3 + 4);
constexpr int kDkdvProducer = kDkdvEwWarps, kDkdvIssuer = kDkdvEwWarps + 1;   // issuers: +1 and +2
constexpr int kDkdvCopier = kDkdvEwWarps + 3;   // four warps that hand dS^T tiles to the dQ kernel
constexpr int kMaxBlocks = 1024;   // q or kv blocks per sequence (64K tokens)
constexpr int kMaxEntries = 2048;  // list entries per CTA

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// ------------------------------------------------------------------ delta
// The workspace holds two arrays of batch x hq rows, each row padded to whole q blocks:
// -delta first, then -lse * log2(e) (-inf for an empty row, so that P = 0): both enter the
// kernels as addends of packed fp32 operations.  Padding rows get 0 and -inf, which lets the
// dK/dV kernel copy a block's 64 values with one bulk copy.
__host__ __device__ inline int padded_sq(int sq) { return (sq + kBS - 1) / kBS * kBS; }

// Eight lanes per (b, h, i) row of D elements (four rows per warp): a lane reads D/64
// 16-byte pieces of O and of dO, so that every thread has several independent loads in flight.
template <bool BF16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& g) {
  float s = 0.f;
  const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x, y;
    if (BF16) {
      x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av[i]));
      y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv[i]));
    } else {
      x = __half22float2(*reinterpret_cast<const __half2*>(&av[i]));
      y = __half22float2(*reinterpret_cast<const __half2*>(&gv[i]));
    }
    s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
  }
  return s;
}
__device__ __forceinline__ uint4 load16(const uint8_t* p, bool wide) {
  if (wide) return *reinterpret_cast<const uint4*>(p);
  const uint2 a = *reinterpret_cast<const uint2*>(p), b = *reinterpret_cast<const uint2*>(p + 8);
  return make_uint4(a.x, a.y, b.x, b.y);
}

template <bool BF16, int D>
__global__ void bwd_delta_vec_kernel(bsa_bwd_params bp) {
  const bsa_fwd_params& p = bp.f;
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int sp = padded_sq(p.sq);
  const long long w = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 4 + (lane >> 3);
  const long long total = (long long)p.batch * p.hq * sp;
  const bool live = w < total;
  const int i = live ? (int)(w % sp) : 0;
  const int h = live ? (int)((w / sp) % p.hq) : 0;
  const int b = live ? (int)(w / ((long long)sp * p.hq)) : 0;
  const bool real = live && i < p.sq;
  float s = 0.f;
  if (real) {
    const bool wide = reinterpret_cast<uintptr_t>(p.o) % 16 == 0 && p.o_ss % 8 == 0 && p.o_sh % 8 == 0 &&
                      p.o_sb % 8 == 0 && reinterpret_cast<uintptr_t>(bp.d_o) % 16 == 0 &&
                      bp.do_ss % 8 == 0 && bp.do_sh % 8 == 0 && bp.do_sb % 8 == 0;
    const uint8_t* op = reinterpret_cast<const uint8_t*>(p.o) +
                        ((int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)i * p.o_ss) * 2 + sub * 16;
    const uint8_t* gp = reinterpret_cast<const uint8_t*>(bp.d_o) +
                        ((int64_t)b * bp.do_sb + (int64_t)h * bp.do_sh + (int64_t)i * bp.do_ss) * 2 + sub * 16;
    uint4 ov[D / 64], gv[D / 64];
#pragma unroll
    for (int j = 0; j < D / 64; ++j) {
      // D is the kernels' padded width; the rows hold p.d columns
      const bool in = j * 64 + sub * 8 < p.d;
      ov[j] = in ? load16(op + j * 128, wide) : make_uint4(0u, 0u, 0u, 0u);
      gv[j] = in ? load16(gp + j * 128, wide) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < D / 64; ++j) s += dot8<BF16>(ov[j], gv[j]);
  }
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (live && sub == 0) {
    if (!real) {
      bp.delta[w] = 0.f;
      bp.delta[total + w] = -INFINITY;
    } else {
      if (bp.d_lse) s -= bp.d_lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + i];
      bp.delta[w] = -s;
      const float l = p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + i];
      bp.delta[total + w] = l == -INFINITY ? -INFINITY : -l * kLog2e;
    }
  }
}

// ------------------------------------------------------------------ shared list builder
// Ordered union of two sets of block indices given as bitmaps; appended to `list`
// starting at *count.  entry = block | extra | (in set 0) << 24 | (in set 1) << 25.
// wordpos (optional): list position of the first entry of every 32-block word, so that the
// position of a block known to be in the union is wordpos[blk / 32] + popc(lower bits of its word).
__device__ __forceinline__ void append_union(const uint32_t* bits0, const uint32_t* bits1,
                                             uint32_t* list, int* count, uint32_t extra, int lane,
                                             int cap, int* wordpos = nullptr) {
  const uint32_t u0 = bits0[lane], u1 = bits1[lane];
  const uint32_t u = u0 | u1;
  const int cnt = __popc(u);
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const int base = *count;
  const int first = base + incl - cnt;   // list position of this lane's word
  if (wordpos) wordpos[lane] = first;
  // one word at a time; within a word every lane owns one bit
  uint32_t nonzero = __ballot_sync(0xffffffffu, u != 0u);
  while (nonzero) {
    const int w = __ffs(nonzero) - 1;
    nonzero &= nonzero - 1;
    const uint32_t uw = __shfl_sync(0xffffffffu, u, w);
    const uint32_t u0w = __shfl_sync(0xffffffffu, u0, w);
    const uint32_t u1w = __shfl_sync(0xffffffffu, u1, w);
    const int pos = __shfl_sync(0xffffffffu, first, w) + __popc(uw & ((1u << lane) - 1u));
    if (((uw >> lane) & 1u) && pos < cap)
      list[pos] = (uint32_t)(w * 32 + lane) | extra | (((u0w >> lane) & 1u) << 24) |
                  (((u1w >> lane) & 1u) << 25);
  }
  __syncwarp();
  if (lane == 31) *count = min(base + incl, cap);
}

// ------------------------------------------------------------------ dK / dV
constexpr int kQdoStages = 4;
template <int D> struct DkdvGeo {
  static constexpr int kSub = D / 64;                    // 64-dim sub-tiles of [rows][128 bytes]
  static constexpr int kKVResident = 2 * 128 * D * 2;    // K and V tiles (128 kv rows each)
  static constexpr int kQdoTile = kBS * D * 2;           // one Q_r or dO_r tile
  static constexpr int kQdoStageBytes = 2 * kQdoTile;
};

struct DkdvTail {
  uint64_t kv_full;
  uint64_t qdo_full[kQdoStages], qdo_empty[kQdoStages];
  // s_full / dp_full: S^T_e / dP^T_e have completed; pt_full / ds_full: every element-wise warp has
  // stored its part of P^T_e / dS^T_e (and has read S^T_e / dP^T_e before)
  uint64_t s_full[2], dp_full[2], pt_full[2], ds_full[2];
  uint64_t ds_read[2];   // dS hand-over: the copier warps have read dS^T_e out of tensor memory
  uint64_t all_done;
  uint32_t tmem_base;
  int n_list;
  // [stage][0 = -lse*log2e, 1 = -delta][row of the q block]: bulk-copied with the stage's tiles
  alignas(128) float ld[kQdoStages][2][kBS];
  uint32_t bits[2][kMaxBlocks / 32];
  uint32_t list[kMaxEntries];
  // dS hand-over: index in the CSR (= tile of the dS workspace) of the entry's block in either half
  int wordpos[32];
  int32_t cidx[kMaxEntries][2];
};
template <int D> constexpr size_t dkdv_smem() {
  return 1024 + DkdvGeo<D>::kKVResident + kQdoStages * DkdvGeo<D>::kQdoStageBytes + sizeof(DkdvTail);
}

template <bool BF16, int D>
__global__ void __launch_bounds__(kDkdvThreads, 1)
bwd_dkdv_sm100_kernel(const __grid_constant__ Tmap4 tmQ, const __grid_constant__ Tmap4 tmK,
                      const __grid_constant__ Tmap4 tmV, const __grid_constant__ Tmap4 tmDO,
                      bsa_bwd_params bp, int* wait_status) {
  const bsa_fwd_params& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kSub = DkdvGeo<D>::kSub, kKVResident = DkdvGeo<D>::kKVResident;
  constexpr int kQdoTile = DkdvGeo<D>::kQdoTile, kQdoStageBytes = DkdvGeo<D>::kQdoStageBytes;
  uint8_t* sK = smem;                    // [kSub subtiles][128 rows][128 B]
  uint8_t* sV = smem + 128 * D * 2;
  uint8_t* sQdo = smem + kKVResident;    // stage s: Q_r, then dO_r
  DkdvTail* tl = reinterpret_cast<DkdvTail*>(smem + kKVResident + kQdoStages * kQdoStageBytes);

  // The dQ kernel is launched behind this one as a programmatic dependent and reads nothing
  // this kernel writes: its CTAs may become resident as soon as every CTA of this grid has
  // started, and fill the SMs that the last, uneven wave of this grid leaves idle.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (*reinterpret_cast<volatile int*>(wait_status) != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Long tiles first: adjacent pairs are longest at the low (causal) end already, the caller's
  // pairing table lists the pairs by ascending column length.
  const int c2 = bp.kv_pairs ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.hq / p.hkv;
  const int past = p.causal ? p.sk - p.sq : 0;
  // the two kv blocks of this tile: adjacent ones, or the caller's pairing
  int kblk[2] = {2 * c2, 2 * c2 + 1};
  if (bp.kv_pairs) {
    const int32_t* pr = bp.kv_pairs + (int64_t)hk * bp.kv_pairs_sh + 2 * c2;
    kblk[0] = pr[0];
    kblk[1] = pr[1];
  }
  const int kvalid[2] = {kblk[0] >= 0 && kblk[0] * kBS < p.sk ? 1 : 0,
                         kblk[1] >= 0 && kblk[1] * kBS < p.sk ? 1 : 0};
  if (!kvalid[0] && !kvalid[1]) return;
  const int nqb = min((p.sq + kBS - 1) / kBS, kMaxBlocks);
  const int sq_pad = padded_sq(p.sq);
  const int64_t ws_half = (int64_t)p.batch * p.hq * sq_pad;

  if (tid == 0) {
    mbar_init(&tl->kv_full, 1);
    for (int s = 0; s < kQdoStages; ++s) {
      mbar_init(&tl->qdo_full[s], 1);
      mbar_init(&tl->qdo_empty[s], 2);   // both issuers have finished with the stage
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tl->s_full[s], 1);
      mbar_init(&tl->dp_full[s], 1);
      mbar_init(&tl->pt_full[s], kDkdvEwWarps);   // one arrival per element-wise warp
      mbar_init(&tl->ds_full[s], kDkdvEwWarps);
      mbar_init(&tl->ds_read[s], 4);
    }
    mbar_init(&tl->all_done, 2);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ.map);
    tma_prefetch_desc(&tmK.map);
    tma_prefetch_desc(&tmV.map);
    tma_prefetch_desc(&tmDO.map);
    tl->n_list = 0;
  }
  __syncthreads();
  // resident K / V tiles and the TMEM allocation overlap the list construction
  if (warp == kDkdvProducer && lane == 0) {
    mbar_expect_tx(&tl->kv_full, (uint32_t)(kvalid[0] + kvalid[1]) * 2 * (kBS * D * 2));
    for (int t = 0; t < 2; ++t) {
      if (!kvalid[t]) continue;
      for (int c = 0; c < kSub; ++c) {
        tma_load_tile(sK + c * 16384 + t * 8192, &tmK, &tl->kv_full, c * 64, kblk[t] * kBS, hk, b);
        tma_load_tile(sV + c * 16384 + t * 8192, &tmV, &tl->kv_full, c * 64, kblk[t] * kBS, hk, b);
      }
    }
  }
  if (warp == kDkdvIssuer) {
    tmem_alloc(&tl->tmem_base, 512);
    tmem_relinquish();
  }
  // ---- entry list: for every q head of the group, union of the two CSC columns
  for (int g = 0; g < G; ++g) {
    if (tid < 2 * (kMaxBlocks / 32)) (&tl->bits[0][0])[tid] = 0u;
    __syncthreads();
    const int h = hk * G + g;
    const int hp = pattern_head(h, p.h_pat, p.hq, p.hkv);
    const int32_t* cc = bp.ccol + (int64_t)hp * bp.ccol_sh;
    const int32_t* rows = bp.row + (int64_t)hp * bp.row_sh;
    // With the dS hand-over every (entry, half) also needs the block's index in the CSR: it is
    // fetched together with the row (a column has at most kMaxBlocks rows, i.e. at most kKeep per
    // thread) and stored once the row's list position is known.
    constexpr int kKeep = (kMaxBlocks + kDkdvThreads - 1) / kDkdvThreads;
    int keep_r[2][kKeep], keep_c[2][kKeep];
    const int32_t* c2r = bp.ds_ws ? bp.csc_csr + (int64_t)hp * bp.row_sh : nullptr;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
#pragma unroll
      for (int k = 0; k < kKeep; ++k) keep_r[t][k] = -1;
      if (!kvalid[t] || kblk[t] >= bp.n_cols) continue;
      const int r_beg = cc[kblk[t]], r_end = cc[kblk[t] + 1];
#pragma unroll
      for (int k = 0; k < kKeep; ++k) {
        const int i = r_beg + tid + k * kDkdvThreads;
        if (i >= r_end) continue;
        const int r = rows[i];
        const int ci = c2r ? c2r[i] : 0;
        if (r < 0 || r >= nqb) continue;
        const int q_pos_last = past + min(r * kBS + kBS, p.sq) - 1;
        if (p.causal && kblk[t] * kBS > q_pos_last) continue;
        atomicOr(&tl->bits[t][r >> 5], 1u << (r & 31));
        keep_r[t][k] = r;
        keep_c[t][k] = ci;
      }
    }
    __syncthreads();
    if (warp == 0)
      append_union(tl->bits[0], tl->bits[1], tl->list, &tl->n_list, (uint32_t)g << 16, lane,
                   kMaxEntries, tl->wordpos);
    __syncthreads();
    if (bp.ds_ws) {
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int k = 0; k < kKeep; ++k) {
          const int r = keep_r[t][k];
          if (r < 0) continue;
          const uint32_t u = tl->bits[0][r >> 5] | tl->bits[1][r >> 5];
          const int pos = tl->wordpos[r >> 5] + __popc(u & ((1u << (r & 31)) - 1u));
          // every attended block has a tile of the scratch, and the list holds all entries
          if (BSA_IN_BOUNDS(pos >= 0 && pos < kMaxEntries && keep_c[t][k] >= 0 &&
                                keep_c[t][k] < bp.ds_tiles_per_head, wait_status, 811) &&
              pos < kMaxEntries)
            tl->cidx[pos][t] = keep_c[t][k];
        }
      __syncthreads();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = tl->n_list;
  const uint32_t tmem = tl->tmem_base;
  const uint32_t tST[2] = {tmem, tmem + 64};
  const uint32_t tDP[2] = {tmem + 128, tmem + 192};
  const uint32_t tDV = tmem + 256, tDK = tmem + 256 + D;

  if (n > 0 && warp == kDkdvProducer) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int e = 0; e < n; ++e) {
        const int s = e % kQdoStages;
        const uint32_t ent = tl->list[e];
        const int r = ent & 0xffff, h = hk * G + ((ent >> 16) & 0xff);
        if (!mbar_wait(&tl->qdo_empty[s], ((e / kQdoStages) & 1) ^ 1, wait_status, 301)) break;
        mbar_expect_tx(&tl->qdo_full[s], kQdoStageBytes + 2 * kBS * 4);
        uint8_t* qd = sQdo + s * kQdoStageBytes;
        uint8_t* gd = qd + kQdoTile;
        for (int c = 0; c < kSub; ++c) {
          tma_load_tile(qd + c * 8192, &tmQ, &tl->qdo_full[s], c * 64, r * kBS, h, b);
          tma_load_tile(gd + c * 8192, &tmDO, &tl->qdo_full[s], c * 64, r * kBS, h, b);
        }
        const int64_t row0 = ((int64_t)b * p.hq + h) * sq_pad + (int64_t)r * kBS;
        // the entry's q block lies in the sequence, its 64 lse / delta values in their half of the workspace
        (void)BSA_IN_BOUNDS(r >= 0 && r * kBS < p.sq && h >= 0 && h < p.hq && row0 >= 0 && row0 + kBS <= ws_half,
                            wait_status, 812);
        bulk_load(tl->ld[s][0], bp.delta + ws_half + row0, kBS * 4, &tl->qdo_full[s]);
        bulk_load(tl->ld[s][1], bp.delta + row0, kBS * 4, &tl->qdo_full[s]);
      }
    }
  } else if (n > 0 && (warp == kDkdvIssuer || warp == kDkdvIssuer + 1)) {
    // ------------------------------------------------------------ MMA issuers
    // A tcgen05.mma costs its issuing thread about as long as a 128x64x16 product takes on
    // the tensor pipe, so the 24 products of an entry are shared by two warps, split by data
    // path rather than by stage:
    //   path 0:  S^T_e = K Q_e^T     ->  P^T_e   ->  dV += P^T_e dO_e
    //   path 1:  dP^T_e = V dO_e^T   ->  dS^T_e  ->  dK += dS^T_e Q_e
    // Each warp issues the first stage of entries 0 and 1, then per entry e its second stage
    // followed at once by the first stage of entry e+2, which overwrites the columns the
    // second stage reads: the tensor pipe executes one thread's products in issue order, so
    // no completion has to be waited for in between, and every such hazard stays inside one
    // warp.  The warps run converged (descriptors stay in uniform registers); only the
    // tcgen05 instructions sit under the elected lane.
    {
      const int path = warp - kDkdvIssuer;
      const uint32_t idesc_nt = umma_idesc(BF16, 128, kBS, false, false);
      const uint32_t idesc_acc = umma_idesc(BF16, 128, D, false, true);
      // first stage: A = resident K (path 0) or V (path 1); B = Q_e or dO_e, K-major
      const uint64_t adesc = umma_desc_sw128(smem_u32(path ? sV : sK), 16, 1024);
      const uint64_t bdesc0 = umma_desc_sw128(smem_u32(sQdo) + (path ? kQdoTile : 0), 16, 1024);
      // second stage: B = dO_e (path 0) or Q_e (path 1) read MN-major: 16 q rows (2 KB) per
      // k-step, the two 64-dim halves 8 KB apart
      const uint64_t mdesc0 = umma_desc_sw128(smem_u32(sQdo) + (path ? 0 : kQdoTile), 8192, 1024);
      const uint32_t tFirst[2] = {path ? tDP[0] : tST[0], path ? tDP[1] : tST[1]};
      const uint32_t tAcc = path ? tDK : tDV;
      auto first_stage = [&](int e) -> bool {
        const int s = e % kQdoStages, bf = e & 1;
        if (!mbar_wait(&tl->qdo_full[s], (e / kQdoStages) & 1, wait_status, 303)) return false;
        tc_fence_after();
        const uint64_t bd = bdesc0 + (uint64_t)((s * kQdoStageBytes) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i)   // i = c * 4 + kk
            tc_mma_ss(tFirst[bf], adesc + (uint64_t)(((i >> 2) * 16384 + (i & 3) * 32) >> 4),
                      bd + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_nt, i ? 1u : 0u);
          tc_commit(path ? &tl->dp_full[bf] : &tl->s_full[bf]);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait(&tl->kv_full, 0, wait_status, 302);
      for (int e = 0; e < 2 && e < n && ok; ++e) ok = first_stage(e);
      for (int e = 0; e < n && ok; ++e) {
        const int s = e % kQdoStages, bf = e & 1;
        if (!mbar_wait(path ? &tl->ds_full[bf] : &tl->pt_full[bf], (e >> 1) & 1, wait_status, 304)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t md = mdesc0 + (uint64_t)((s * kQdoStageBytes) >> 4);
        const uint32_t acc0 = e ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_ts(tAcc, tFirst[bf] + kk * 16, md + (uint64_t)((kk * 2048) >> 4), idesc_acc,
                      kk ? 1u : acc0);
          tc_commit(&tl->qdo_empty[s]);
        }
        __syncwarp();
        // dP^T of entry e+2 overwrites dS^T_e: with the dS hand-over the copier warps must have read it
        if (path == 1 && bp.ds_ws && e + 2 < n &&
            !mbar_wait(&tl->ds_read[bf], (e >> 1) & 1, wait_status, 310)) {
          ok = false;
          break;
        }
        if (e + 2 < n) ok = first_stage(e + 2);
      }
      if (ok && elect_one()) tc_commit(&tl->all_done);
    }
    __syncwarp();
  } else if (n > 0 && warp >= kDkdvCopier) {
    // ------------------------------------------------------------ dS hand-over (four warps)
    // One warp per TMEM lane quadrant reads the packed dS^T rows of an entry (64 q columns =
    // 128 bytes per kv row, in the first 8 of every 16 columns) once the element-wise warps have
    // stored them, releases the columns, and writes the attended half's tile for the dQ kernel as
    // eight slabs of [64 kv rows][8 q columns] (16 bytes per row): the warp's 32 kv rows are
    // contiguous within a slab, so every store instruction is one 512-byte run, and a slab is a
    // column of the 8 x 16-byte core matrices the tensor core reads without swizzle.  The
    // element-wise warps, whose time per entry sets the pace of this kernel, do none of this.
    if (bp.ds_ws) {
      const int quad = warp & 3, t = quad >> 1;
      const int rk = (quad & 1) * 32 + lane;   // kv row inside the half's block
      const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
      for (int e = 0; e < n; ++e) {
        if (!mbar_wait(&tl->ds_full[e & 1], (e >> 1) & 1, wait_status, 323)) break;
        tc_fence_after();
        const uint32_t ent = tl->list[e];
        const bool att_blk = ((ent >> (24 + t)) & 1u) != 0 && kvalid[t];
        uint32_t w[32];
        if (att_blk) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tmem_ld8(tDP[e & 1] + lane_off + j * 16, *reinterpret_cast<uint32_t(*)[8]>(&w[8 * j]));
          tmem_ld_wait();
        }
        tc_fence_before();
        __syncwarp();
        // relaxed: the loads have completed (wait::ld) and nothing is published; a release would
        // wait for the previous entry's stores
        if (lane == 0) mbar_arrive_relaxed(&tl->ds_read[e & 1]);
        if (att_blk) {
          const int h = hk * G + (int)((ent >> 16) & 0xffu);
          const int64_t tile = ((int64_t)b * p.hq + h) * bp.ds_tiles_per_head + tl->cidx[e][t];
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(bp.ds_ws) + tile * 8192) + rk;
          if (BSA_IN_BOUNDS(tl->cidx[e][t] >= 0 && tl->cidx[e][t] < bp.ds_tiles_per_head && h < p.hq, wait_status, 813)) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              __stcs(dst + j * kBS, make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
          }
        }
      }
    }
  } else if (n > 0 && warp < kDkdvEwWarps) {
    // ------------------------------------------------------------ P^T / dS^T (warps 0-15)
    // A warp owns a TMEM lane quadrant (32 kv rows) and 16 of the 64 q columns; its packed
    // 16-bit results overwrite the first 8 of the 16 fp32 columns it has just read, so the
    // second-stage k-step kk (16 q rows) starts at column 16 kk.
    const int quad = warp & 3, qtr = warp >> 2;
    const int r_kv = quad * 32 + lane;             // tile row = TMEM lane
    const int t = r_kv >> 6;
    const int kpos = kblk[t] * kBS + (r_kv & 63);
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    const uint64_t scale_2 = f32x2(scale2, scale2);
    bool alive = true;
    for (int e = 0; e < n; ++e) {
      const int st = e % kQdoStages;
      // the stage's lse / delta rows arrive with its tiles
      if (!mbar_wait(&tl->qdo_full[st], (e / kQdoStages) & 1, wait_status, 309)) { alive = false; break; }
      if (!mbar_wait(&tl->s_full[e & 1], (e >> 1) & 1, wait_status, 305)) { alive = false; break; }
      tc_fence_after();
      const uint32_t ent = tl->list[e];
      const int r = ent & 0xffff;
      const bool att_blk = ((ent >> (24 + t)) & 1u) != 0 && kvalid[t];   // the same for the whole warp
      const bool att = att_blk && kpos < p.sk;   // rows past the end of the keys hold P = dS = 0
      // causal: q position past + r*64 + c must be >= kpos  ->  c >= c0
      const int c0 = (p.causal ? kpos - past - r * kBS : 0) - qtr * 16;
      const float* lse_s = tl->ld[st][0] + qtr * 16;
      const float* del_s = tl->ld[st][1] + qtr * 16;
      // P^T is published as soon as S^T allows it, while dP^T_e may still be on the tensor pipe:
      // dV += P^T dO and the S^T of entry e+2 behind it then start without waiting for dS^T.
      uint32_t sv[16];
      tmem_ld16(tST[e & 1] + lane_off + qtr * 16, sv);
      tmem_ld_wait();
      uint64_t pv2[8];   // P as packed fp32 pairs, kept for dS
      uint32_t pp[8];
      if (att) {
        // only a diagonal entry has masked columns: they get S = -inf, hence P = dS = 0
        if (c0 > 0) {
#pragma unroll
          for (int c = 0; c < 16; ++c)
            if (c < c0) sv[c] = 0xff800000u;
        }
        if (p.fine_block) {
          // a pattern with 16- or 32-token blocks, coarsened: bit a * (64 / fb) + b of the entry's mask
          // says whether q sub-block a attends kv sub-block b (this thread: one kv row, 16 q columns)
          const int sh = p.fine_block == 16 ? 4 : 5, kf = 64 >> sh;
          const int hq_ = hk * G + (int)((ent >> 16) & 0xffu);
          const uint32_t bits = (uint32_t)__ldg(p.col_bits + (int64_t)pattern_head(hq_, p.h_pat, p.hq, p.hkv) *
                                                             p.col_bits_sh + tl->cidx[e][t]) >>
                                ((r_kv & 63) >> sh);
#pragma unroll
          for (int c = 0; c < 16; ++c)
            if (!((bits >> (((qtr * 16 + c) >> sh) * kf)) & 1u)) sv[c] = 0xff800000u;
        }
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c4 * 4);
          // two columns per instruction: P = exp2(S c - lse)
          const uint64_t nl[2] = {f32x2(l4.x, l4.y), f32x2(l4.z, l4.w)};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            float x0, x1;
            f32x2_split(fma_f32x2(f32x2(sv[c4 * 4 + 2 * i], sv[c4 * 4 + 2 * i + 1]), scale_2, nl[i]), x0, x1);
            const float p0 = ex2(x0), p1 = ex2(x1);
            pv2[c4 * 2 + i] = f32x2(p0, p1);
            pp[c4 * 2 + i] = pack2<BF16>(p0, p1);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { pp[i] = 0u; pv2[i] = 0ull; }
      }
      tmem_st8(tST[e & 1] + lane_off + qtr * 16, pp);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->pt_full[e & 1]);
      if (!mbar_wait(&tl->dp_full[e & 1], (e >> 1) & 1, wait_status, 307)) { alive = false; break; }
      tc_fence_after();
      uint32_t dv[16], ds[8];
      tmem_ld16(tDP[e & 1] + lane_off + qtr * 16, dv);
      tmem_ld_wait();
      if (att) {
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const float4 d4 = *reinterpret_cast<const float4*>(del_s + c4 * 4);
          const uint64_t nd[2] = {f32x2(d4.x, d4.y), f32x2(d4.z, d4.w)};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            // dS = P (dP - delta)
            float d0, d1;
            f32x2_split(mul_f32x2(pv2[c4 * 2 + i],
                                  add_f32x2(f32x2(dv[c4 * 4 + 2 * i], dv[c4 * 4 + 2 * i + 1]), nd[i])), d0, d1);
            ds[c4 * 2 + i] = pack2<BF16>(d0, d1);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) ds[i] = 0u;
      }
      tmem_st8(tDP[e & 1] + lane_off + qtr * 16, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->ds_full[e & 1]);
    }
    // ---- epilogue: warp = (lane quadrant, dV or dK, 64-column half); every thread scales
    // its row and stores 128 contiguous bytes straight from registers
    if (alive) alive = mbar_wait(&tl->all_done, 0, wait_status, 306);
    tc_fence_after();
    if (alive) {
      const int is_dk = (warp >> 2) & 1, ch0 = (warp >> 3) * (D / 64);
      const int kv = kblk[t] * kBS + (r_kv & 63);
      const bool row_ok = kvalid[t] && kv < p.sk && BSA_IN_BOUNDS(kv >= 0 && hk < p.hkv && b < p.batch, wait_status, 814);
      void* gbase = is_dk ? bp.dk : bp.dv;
      const int64_t sb = is_dk ? bp.dk_sb : bp.dv_sb, sh = is_dk ? bp.dk_sh : bp.dv_sh,
                    ss = is_dk ? bp.dk_ss : bp.dv_ss;
      uint8_t* grow = reinterpret_cast<uint8_t*>(gbase) + ((int64_t)b * sb + (int64_t)hk * sh + (int64_t)kv * ss) * 2;
      const bool wide = reinterpret_cast<uintptr_t>(gbase) % 16 == 0 && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0;
      const float scale = is_dk ? p.sm_scale : 1.f;
      const uint32_t tacc = is_dk ? tDK : tDV;
#pragma unroll
      for (int ch = ch0; ch < ch0 + D / 64; ++ch) {
        uint32_t o[32];
        tmem_ld32(tacc + lane_off + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * scale, __uint_as_float(o[2 * i + 1]) * scale);
        if (row_ok) {
          if (wide) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (ch * 32 + i * 8 < p.d)   // columns at or past the real head dim are padding
                *reinterpret_cast<uint4*>(grow + ch * 64 + i * 16) =
                    make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (ch * 32 + i * 4 < p.d)
                *reinterpret_cast<uint2*>(grow + ch * 64 + i * 8) = make_uint2(w[2 * i], w[2 * i + 1]);
          }
        }
      }
    }
  } else if (warp == kDkdvProducer) {
    if (lane == 0) mbar_wait(&tl->kv_full, 0, wait_status, 308);   // let the tiles in flight land
  } else if (warp < 4) {
    // nothing attends these kv blocks: zero gradients
    const int t = tid >> 6;
    const int kv = kblk[t] * kBS + (tid & 63);
    if (kvalid[t] && kv < p.sk) {
      uint2* d1 = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(bp.dk) +
          ((int64_t)b * bp.dk_sb + (int64_t)hk * bp.dk_sh + (int64_t)kv * bp.dk_ss) * 2);
      uint2* d2 = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(bp.dv) +
          ((int64_t)b * bp.dv_sb + (int64_t)hk * bp.dv_sh + (int64_t)kv * bp.dv_ss) * 2);
      for (int i = 0; i < p.d / 4; ++i) { d1[i] = make_uint2(0u, 0u); d2[i] = make_uint2(0u, 0u); }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kDkdvIssuer) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------ dQ
constexpr int kDqKStages = 3, kDqVStages = 2;
enum { kPairHeads = 0, kPairRows = 1 };

struct DqTail {
  uint64_t q_full;
  uint64_t k_full[kDqKStages], k_empty[kDqKStages];
  uint64_t v_full[kDqVStages], v_empty[kDqVStages];
  // s_full / dp_full: S_e / dP_e have completed; s_free: every element-wise warp has read S_e;
  // p_full: every element-wise warp has stored its part of dS_e
  uint64_t s_full[2], dp_full[2], s_free[2], p_full[2];
  uint64_t cp_done, all_done;
  uint32_t tmem_base;
  int n_list;
  uint32_t bits[2][kMaxBlocks / 32];
  uint32_t list[kMaxBlocks];
};
template <int D> constexpr size_t dq_smem() {
  return 1024 + 2 * 128 * D * 2 + (kDqKStages + kDqVStages) * (kBS * D * 2) + sizeof(DqTail);
}

template <bool BF16, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_sm100_kernel(const __grid_constant__ Tmap4 tmQ, const __grid_constant__ Tmap4 tmK,
                    const __grid_constant__ Tmap4 tmV, const __grid_constant__ Tmap4 tmDO,
                    bsa_bwd_params bp, int mode, int* wait_status) {
  const bsa_fwd_params& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kSub = D / 64, kTileKV = kBS * D * 2;
  uint8_t* sQ = smem;                       // [kSub subtiles][128 rows][128 B]
  uint8_t* sDO = smem + 128 * D * 2;
  uint8_t* sKs = smem + 2 * 128 * D * 2;    // K stages
  uint8_t* sVs = sKs + kDqKStages * kTileKV;
  DqTail* tl = reinterpret_cast<DqTail*>(sVs + kDqVStages * kTileKV);

  // Launched as a programmatic dependent of the dK/dV kernel, whose results it does not read
  // (a no-op after a plain launch).  No CTA leaves before that grid has completed, so that
  // whatever follows this kernel in the stream also follows the dK/dV kernel.
  auto wait_for_dkdv = [] { asm volatile("griddepcontrol.wait;" ::: "memory"); };
  if (*reinterpret_cast<volatile int*>(wait_status) != 0) { wait_for_dkdv(); return; }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.hq / p.hkv;
  const int b = blockIdx.z;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int past = p.causal ? p.sk - p.sq : 0;
  int head[2], qblk[2], valid[2], kvh;
  if (mode == kPairHeads) {
    const int pairs = G / 2;
    kvh = blockIdx.y / pairs;
    head[0] = kvh * G + 2 * (blockIdx.y % pairs);
    head[1] = head[0] + 1;
    qblk[0] = qblk[1] = tile;
    valid[0] = valid[1] = 1;
  } else {
    head[0] = head[1] = blockIdx.y;
    kvh = blockIdx.y / G;
    qblk[0] = 2 * tile;
    qblk[1] = 2 * tile + 1;
    valid[0] = 1;
    valid[1] = qblk[1] * kBS < p.sq ? 1 : 0;
  }
  if (qblk[0] * kBS >= p.sq) { wait_for_dkdv(); return; }
  const int nkb = min((p.sk + kBS - 1) / kBS, kMaxBlocks);

  if (tid == 0) {
    mbar_init(&tl->q_full, 1);
    // a K stage is read by both issuers (S and dQ), a V stage by one (dP)
    for (int s = 0; s < kDqKStages; ++s) { mbar_init(&tl->k_full[s], 1); mbar_init(&tl->k_empty[s], 2); }
    for (int s = 0; s < kDqVStages; ++s) { mbar_init(&tl->v_full[s], 1); mbar_init(&tl->v_empty[s], 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tl->s_full[s], 1);
      mbar_init(&tl->dp_full[s], 1);
      mbar_init(&tl->s_free[s], kDqEwWarps);   // one arrival per element-wise warp
      mbar_init(&tl->p_full[s], kDqEwWarps);
    }
    mbar_init(&tl->cp_done, 1);
    mbar_init(&tl->all_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ.map);
    tma_prefetch_desc(&tmK.map);
    tma_prefetch_desc(&tmV.map);
    tma_prefetch_desc(&tmDO.map);
    tl->n_list = 0;
  }
  if (tid < 2 * (kMaxBlocks / 32)) (&tl->bits[0][0])[tid] = 0u;
  __syncthreads();
  if (warp == kWarpProducer && lane == 0) {
    mbar_expect_tx(&tl->q_full, (uint32_t)(valid[0] + valid[1]) * 2 * (kBS * D * 2));
    for (int t = 0; t < 2; ++t) {
      if (!valid[t]) continue;
      for (int c = 0; c < kSub; ++c) {
        tma_load_tile(sQ + c * 16384 + t * 8192, &tmQ, &tl->q_full, c * 64, qblk[t] * kBS, head[t], b);
        tma_load_tile(sDO + c * 16384 + t * 8192, &tmDO, &tl->q_full, c * 64, qblk[t] * kBS, head[t], b);
      }
    }
  }
  if (warp == kWarpIssueA) {
    tmem_alloc(&tl->tmem_base, 512);
    tmem_relinquish();
  }
  for (int t = 0; t < 2; ++t) {
    if (!valid[t] || qblk[t] >= p.n_rows) continue;
    const int hp = pattern_head(head[t], p.h_pat, p.hq, p.hkv);
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
    const int c_beg = cr[qblk[t]], c_end = cr[qblk[t] + 1];
    const int q_pos_last = past + min(qblk[t] * kBS + kBS, p.sq) - 1;
    for (int i = c_beg + tid; i < c_end; i += kBwdThreads) {
      const int blk = cols[i];
      if (blk >= 0 && blk < nkb && !(p.causal && blk * kBS > q_pos_last))
        atomicOr(&tl->bits[t][blk >> 5], 1u << (blk & 31));
    }
  }
  __syncthreads();
  if (warp == 0) append_union(tl->bits[0], tl->bits[1], tl->list, &tl->n_list, 0u, lane, kMaxBlocks);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = tl->n_list;
  const uint32_t tmem = tl->tmem_base;
  const uint32_t tS[2] = {tmem, tmem + 64};
  const uint32_t tDP[2] = {tmem + 128, tmem + 192};
  const uint32_t tDQ = tmem + 256;
  // Q and dO are the A operands of every first-stage product: they are copied once
  // from their TMA tiles into TMEM (D/2 columns each), which takes them off the
  // shared-memory read path that the tensor pipe saturates.
  const uint32_t tQ = tmem + 256 + D, tDO = tQ + D / 2;

  if (n > 0 && warp == kWarpProducer) {
    if (lane == 0) {
      for (int e = 0; e < n; ++e) {
        const int tok = (int)(tl->list[e] & 0xffffu) * kBS;
        const int sk_ = e % kDqKStages, sv_ = e % kDqVStages;
        if (!mbar_wait(&tl->k_empty[sk_], ((e / kDqKStages) & 1) ^ 1, wait_status, 311)) break;
        mbar_expect_tx(&tl->k_full[sk_], kTileKV);
        for (int c = 0; c < kSub; ++c)
          tma_load_tile(sKs + sk_ * kTileKV + c * 8192, &tmK, &tl->k_full[sk_], c * 64, tok, kvh, b);
        if (!mbar_wait(&tl->v_empty[sv_], ((e / kDqVStages) & 1) ^ 1, wait_status, 312)) break;
        mbar_expect_tx(&tl->v_full[sv_], kTileKV);
        for (int c = 0; c < kSub; ++c)
          tma_load_tile(sVs + sv_ * kTileKV + c * 8192, &tmV, &tl->v_full[sv_], c * 64, tok, kvh, b);
      }
    }
  } else if (n > 0 && warp == kWarpIssueA) {
    // ------------------------------------------------------------ S = Q K^T
    // The products of an entry are shared by two issuer warps along the data paths: this one
    // copies Q and dO into TMEM and issues S_e; the other issues dP_e = dO V_e^T and
    // dQ += dS_e K_e, so that dP_{e+2}, which overwrites the columns dS_e sits in, follows
    // dQ_e in one thread's issue order and needs no completion wait.  The warps run
    // converged; only the tcgen05 instructions sit under the elected lane.
    {
      const uint32_t idesc_nt = umma_idesc(BF16, 128, kBS, false, false);
      const uint64_t qdesc = umma_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t gdesc = umma_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t kdesc0 = umma_desc_sw128(smem_u32(sKs), 16, 1024);
      bool ok = mbar_wait(&tl->q_full, 0, wait_status, 313);
      if (ok) {
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {   // one k-step (16 head dims = 8 packed columns) per copy
            const uint64_t off = (uint64_t)(((i >> 2) * 16384 + (i & 3) * 32) >> 4);
            tc_cp_128x256b(tQ + i * 8, qdesc + off);
            tc_cp_128x256b(tDO + i * 8, gdesc + off);
          }
          tc_commit(&tl->cp_done);
        }
        __syncwarp();
      }
      for (int e = 0; e < n && ok; ++e) {
        const int sk_ = e % kDqKStages, bf = e & 1;
        // S[bf] is free once the element-wise warps have read entry e-2
        if (e >= 2 && !mbar_wait(&tl->s_free[bf], ((e - 2) >> 1) & 1, wait_status, 319)) break;
        if (!mbar_wait(&tl->k_full[sk_], (e / kDqKStages) & 1, wait_status, 314)) break;
        tc_fence_after();
        const uint64_t kd = kdesc0 + (uint64_t)((sk_ * kTileKV) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i)   // i = c * 4 + kk
            tc_mma_ts(tS[bf], tQ + i * 8, kd + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_nt,
                      i ? 1u : 0u);
          tc_commit(&tl->k_empty[sk_]);
          tc_commit(&tl->s_full[bf]);
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (n > 0 && warp == kWarpIssueB) {
    // ------------------------------------------------------------ dP = dO V^T, dQ += dS K
    {
      const uint32_t idesc_nt = umma_idesc(BF16, 128, kBS, false, false);
      const uint32_t idesc_acc = umma_idesc(BF16, 128, D, false, true);
      const uint64_t vdesc0 = umma_desc_sw128(smem_u32(sVs), 16, 1024);
      // B = K_j read MN-major: 16 kv rows (2 KB) per k-step, 64-dim halves 8 KB apart
      const uint64_t kdesc0 = umma_desc_sw128(smem_u32(sKs), 8192, 1024);
      auto issue_dp = [&](int e) -> bool {
        const int sv_ = e % kDqVStages, bf = e & 1;
        if (!mbar_wait(&tl->v_full[sv_], (e / kDqVStages) & 1, wait_status, 315)) return false;
        tc_fence_after();
        const uint64_t vd = vdesc0 + (uint64_t)((sv_ * kTileKV) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i)
            tc_mma_ts(tDP[bf], tDO + i * 8, vd + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_nt,
                      i ? 1u : 0u);
          tc_commit(&tl->v_empty[sv_]);
          tc_commit(&tl->dp_full[bf]);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait(&tl->cp_done, 0, wait_status, 318);   // dO is in TMEM
      for (int e = 0; e < 2 && e < n && ok; ++e) ok = issue_dp(e);
      for (int e = 0; e < n && ok; ++e) {
        const int sk_ = e % kDqKStages, bf = e & 1;
        if (!mbar_wait(&tl->p_full[bf], (e >> 1) & 1, wait_status, 316)) { ok = false; break; }
        if (!mbar_wait(&tl->k_full[sk_], (e / kDqKStages) & 1, wait_status, 321)) { ok = false; break; }
        tc_fence_after();
        const uint64_t kd = kdesc0 + (uint64_t)((sk_ * kTileKV) >> 4);
        const uint32_t acc0 = e ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_ts(tDQ, tDP[bf] + kk * 16, kd + (uint64_t)((kk * 2048) >> 4), idesc_acc,
                      kk ? 1u : acc0);
          tc_commit(&tl->k_empty[sk_]);
        }
        __syncwarp();
        if (e + 2 < n) ok = issue_dp(e + 2);
      }
      if (ok && elect_one()) tc_commit(&tl->all_done);
    }
    __syncwarp();
  } else if (n > 0 && warp < kDqEwWarps) {
    // ------------------------------------------------------------ dS (warps 0-15)
    // A warp owns a TMEM lane quadrant (32 q rows) and 16 of the 64 kv columns; its packed dS
    // overwrites the first 8 of the 16 dP columns it has read, so k-step kk of dQ += dS K
    // starts at column 16 kk.
    const int quad = warp & 3, qtr = warp >> 2;
    const int r = quad * 32 + lane, t = r >> 6, rr = r & 63;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    const int q_row = qblk[t] * kBS + rr;
    const int qpos = past + q_row;
    float neg_lse = -INFINITY, neg_delta = 0.f;
    if (valid[t] && q_row < p.sq) {
      const float l = p.lse[(int64_t)b * p.lse_sb + (int64_t)head[t] * p.lse_sh + q_row];
      neg_lse = l == -INFINITY ? -INFINITY : -l * kLog2e;
      neg_delta = bp.delta[((int64_t)b * p.hq + head[t]) * padded_sq(p.sq) + q_row];   // holds -delta
    }
    const uint64_t scale_2 = f32x2(scale2, scale2), neg_lse2 = f32x2(neg_lse, neg_lse),
                   neg_delta2 = f32x2(neg_delta, neg_delta);
    bool alive = true;
    for (int e = 0; e < n; ++e) {
      if (!mbar_wait(&tl->s_full[e & 1], (e >> 1) & 1, wait_status, 317)) { alive = false; break; }
      tc_fence_after();
      const uint32_t ent = tl->list[e];
      const int kbase = (int)(ent & 0xffffu) * kBS;
      const bool att = ((ent >> (24 + t)) & 1u) != 0 && valid[t];
      int lim = p.sk - kbase;
      if (p.causal) lim = min(lim, qpos - kbase + 1);
      lim -= qtr * 16;   // relative to this warp's 16 columns
      // The exponentials run as soon as S_e is there, while dP_e may still be on the tensor pipe,
      // and S's columns are handed back for entry e+2 right after they have been read.
      uint32_t sv[16];
      tmem_ld16(tS[e & 1] + lane_off + qtr * 16, sv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->s_free[e & 1]);
      uint64_t pv2[8];   // P as packed fp32 pairs
      if (att) {
        // only blocks on the diagonal or at the end of the keys have masked columns:
        // they get S = -inf, hence P = dS = 0
        if (lim < 16) {
#pragma unroll
          for (int c = 0; c < 16; ++c)
            if (c >= lim) sv[c] = 0xff800000u;
        }
#pragma unroll
        for (int c2 = 0; c2 < 8; ++c2) {
          // two columns per instruction: P = exp2(S c - lse)
          float x0, x1;
          f32x2_split(fma_f32x2(f32x2(sv[2 * c2], sv[2 * c2 + 1]), scale_2, neg_lse2), x0, x1);
          pv2[c2] = f32x2(ex2(x0), ex2(x1));
        }
      }
      if (!mbar_wait(&tl->dp_full[e & 1], (e >> 1) & 1, wait_status, 322)) { alive = false; break; }
      tc_fence_after();
      uint32_t dv[16], ds[8];
      tmem_ld16(tDP[e & 1] + lane_off + qtr * 16, dv);
      tmem_ld_wait();
      if (att) {
#pragma unroll
        for (int c2 = 0; c2 < 8; ++c2) {
          // dS = P (dP - delta)
          float d0, d1;
          f32x2_split(mul_f32x2(pv2[c2], add_f32x2(f32x2(dv[2 * c2], dv[2 * c2 + 1]), neg_delta2)), d0, d1);
          ds[c2] = pack2<BF16>(d0, d1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) ds[i] = 0u;
      }
      tmem_st8(tDP[e & 1] + lane_off + qtr * 16, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->p_full[e & 1]);
    }
    // ---- epilogue: warp = (lane quadrant, 32-column chunk); every thread scales its row and
    // stores 64 contiguous bytes straight from registers
    if (alive) alive = mbar_wait(&tl->all_done, 0, wait_status, 318);
    tc_fence_after();
    if (alive && qtr < D / 32) {
      const bool row_ok = valid[t] && q_row < p.sq;
      uint8_t* grow = reinterpret_cast<uint8_t*>(bp.dq) +
                      ((int64_t)b * bp.dq_sb + (int64_t)head[t] * bp.dq_sh + (int64_t)q_row * bp.dq_ss) * 2 +
                      qtr * 64;
      const bool wide = reinterpret_cast<uintptr_t>(bp.dq) % 16 == 0 && bp.dq_sb % 8 == 0 &&
                        bp.dq_sh % 8 == 0 && bp.dq_ss % 8 == 0;
      uint32_t o[32];
      tmem_ld32(tDQ + lane_off + qtr * 32, o);
      tmem_ld_wait();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * p.sm_scale, __uint_as_float(o[2 * i + 1]) * p.sm_scale);
      if (row_ok) {
        if (wide) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (qtr * 32 + i * 8 < p.d)   // columns at or past the real head dim are padding
              *reinterpret_cast<uint4*>(grow + i * 16) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (qtr * 32 + i * 4 < p.d)
              *reinterpret_cast<uint2*>(grow + i * 8) = make_uint2(w[2 * i], w[2 * i + 1]);
        }
      }
    }
  } else if (warp == kWarpProducer) {
    if (lane == 0) mbar_wait(&tl->q_full, 0, wait_status, 320);   // let the tiles in flight land
  } else if (warp < 4) {
    const int t = tid >> 6;
    const int q_row = qblk[t] * kBS + (tid & 63);
    if (valid[t] && q_row < p.sq) {
      uint2* d = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(bp.dq) +
          ((int64_t)b * bp.dq_sb + (int64_t)head[t] * bp.dq_sh + (int64_t)q_row * bp.dq_ss) * 2);
      for (int i = 0; i < p.d / 4; ++i) d[i] = make_uint2(0u, 0u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpIssueA) tmem_dealloc(tmem, 512);
  wait_for_dkdv();
}

// ------------------------------------------------------------------ dQ from handed-over dS
// With a dS workspace the dK/dV kernel has stored the dS^T tile (64 kv rows x 64 q columns, 8 KB, as
// eight slabs of [64 kv rows][8 q columns]) of every attended block at the block's CSR index, and
// dQ needs one product per block,
// dQ += dS K, instead of the three of the kernel above (S and dP again, then dQ): no
// element-wise work, no Q / dO / V / lse / delta.  One CTA per 128-row query tile as above
// (two 64-row halves, union of the halves' CSR rows); per entry the producer warp loads the K
// block and the attended halves' dS^T tiles (a half that does not attend the block gets zeros)
// (plain 8 KB bulk copies) and the issuer runs four SS products with both operands MN-major
// (dS^T: q contiguous, K: head dim contiguous).  Two CTAs per SM (D columns of TMEM each).  The kernel is bound by the
// L2 -> SM traffic of its operands (32 KB per entry against 256 tensor-pipe cycles).
constexpr int kDqsStages = 3;
constexpr int kDqsThreads = 192;   // warps 0-3 epilogue, 4 producer, 5 issuer
constexpr int kDqsProducer = 4, kDqsIssuer = 5;

struct DqsTail {
  uint64_t full[kDqsStages], empty[kDqsStages];
  uint64_t all_done;
  uint32_t tmem_base;
  int n_list;
  int wordpos[32];
  uint32_t bits[2][kMaxBlocks / 32];
  uint32_t list[kMaxBlocks];
  int32_t cidx[kMaxBlocks][2];
};
template <int D> constexpr size_t dqs_smem() {
  return 1024 + kDqsStages * (2 * 8192 + kBS * D * 2) + sizeof(DqsTail);
}

template <bool BF16, int D>
__global__ void __launch_bounds__(kDqsThreads, 2)
bwd_dq_from_ds_kernel(const __grid_constant__ Tmap4 tmK, bsa_bwd_params bp, int mode, int* wait_status) {
  const bsa_fwd_params& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kSub = D / 64, kTileKV = kBS * D * 2, kStageBytes = 2 * 8192 + kTileKV;
  DqsTail* tl = reinterpret_cast<DqsTail*>(smem + kDqsStages * kStageBytes);

  // Programmatic dependent of the dK/dV kernel, whose dS tiles it reads: everything up to the
  // block list is built while that grid drains, the loads start after it has completed.
  auto wait_for_dkdv = [] { asm volatile("griddepcontrol.wait;" ::: "memory"); };
  if (*reinterpret_cast<volatile int*>(wait_status) != 0) { wait_for_dkdv(); return; }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.hq / p.hkv;
  const int b = blockIdx.z;
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int past = p.causal ? p.sk - p.sq : 0;
  int head[2], qblk[2], valid[2], kvh;
  if (mode == kPairHeads) {
    const int pairs = G / 2;
    kvh = blockIdx.y / pairs;
    head[0] = kvh * G + 2 * (blockIdx.y % pairs);
    head[1] = head[0] + 1;
    qblk[0] = qblk[1] = tile;
    valid[0] = valid[1] = 1;
  } else {
    head[0] = head[1] = blockIdx.y;
    kvh = blockIdx.y / G;
    qblk[0] = 2 * tile;
    qblk[1] = 2 * tile + 1;
    valid[0] = 1;
    valid[1] = qblk[1] * kBS < p.sq ? 1 : 0;
  }
  if (qblk[0] * kBS >= p.sq) { wait_for_dkdv(); return; }
  const int nkb = min((p.sk + kBS - 1) / kBS, kMaxBlocks);

  if (tid == 0) {
    for (int s = 0; s < kDqsStages; ++s) { mbar_init(&tl->full[s], 1); mbar_init(&tl->empty[s], 1); }
    mbar_init(&tl->all_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmK.map);
    tl->n_list = 0;
  }
  if (tid < 2 * (kMaxBlocks / 32)) (&tl->bits[0][0])[tid] = 0u;
  __syncthreads();
  if (warp == kDqsIssuer) {
    tmem_alloc(&tl->tmem_base, D);
    tmem_relinquish();
  }
  // block list (as in the kernel above) and, per entry and half, the block's CSR index
  auto for_entries = [&](auto&& fn) {
    for (int t = 0; t < 2; ++t) {
      if (!valid[t] || qblk[t] >= p.n_rows) continue;
      const int hp = pattern_head(head[t], p.h_pat, p.hq, p.hkv);
      const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
      const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
      const int c_beg = cr[qblk[t]], c_end = cr[qblk[t] + 1];
      const int q_pos_last = past + min(qblk[t] * kBS + kBS, p.sq) - 1;
      for (int i = c_beg + tid; i < c_end; i += kDqsThreads) {
        const int blk = cols[i];
        if (blk >= 0 && blk < nkb && !(p.causal && blk * kBS > q_pos_last)) fn(t, blk, i);
      }
    }
  };
  for_entries([&](int t, int blk, int) { atomicOr(&tl->bits[t][blk >> 5], 1u << (blk & 31)); });
  __syncthreads();
  if (warp == 0)
    append_union(tl->bits[0], tl->bits[1], tl->list, &tl->n_list, 0u, lane, kMaxBlocks, tl->wordpos);
  __syncthreads();
  for_entries([&](int t, int blk, int i) {
    const uint32_t u = tl->bits[0][blk >> 5] | tl->bits[1][blk >> 5];
    const int pos = tl->wordpos[blk >> 5] + __popc(u & ((1u << (blk & 31)) - 1u));
    if (BSA_IN_BOUNDS(pos >= 0 && pos < kMaxBlocks && i >= 0 && i < bp.ds_tiles_per_head, wait_status, 815) &&
        pos < kMaxBlocks)
      tl->cidx[pos][t] = i;
  });
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = tl->n_list;
  const uint32_t tmem = tl->tmem_base;
  wait_for_dkdv();

  if (n > 0 && warp == kDqsProducer) {
    // ------------------------------------------------------------ producer (whole warp)
    for (int e = 0; e < n; ++e) {
      const int s = e % kDqsStages;
      if (!mbar_wait(&tl->empty[s], ((e / kDqsStages) & 1) ^ 1, wait_status, 331)) break;
      const uint32_t ent = tl->list[e];
      uint8_t* st = smem + s * kStageBytes;
      const bool a0 = ((ent >> 24) & 1u) != 0 && valid[0], a1 = ((ent >> 25) & 1u) != 0 && valid[1];
      if (!a0 || !a1) {
        // the half that does not attend this block contributes nothing: zeros for its dS^T tile
        uint4* z = reinterpret_cast<uint4*>(st + (a0 ? 8192 : 0));
        for (int i = lane; i < 8192 / 16; i += 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's reads
      }
      __syncwarp();
      if (lane == 0) {
        mbar_expect_tx(&tl->full[s], kTileKV + (uint32_t)((a0 ? 1 : 0) + (a1 ? 1 : 0)) * 8192u);
        const int tok = (int)(ent & 0xffffu) * kBS;
        (void)BSA_IN_BOUNDS(tok < p.sk && kvh < p.hkv && (!a0 || (tl->cidx[e][0] >= 0 && tl->cidx[e][0] < bp.ds_tiles_per_head)) &&
                                (!a1 || (tl->cidx[e][1] >= 0 && tl->cidx[e][1] < bp.ds_tiles_per_head)),
                            wait_status, 816);
        for (int c = 0; c < kSub; ++c)
          tma_load_tile(st + 16384 + c * 8192, &tmK, &tl->full[s], c * 64, tok, kvh, b);
        const uint8_t* ws = reinterpret_cast<const uint8_t*>(bp.ds_ws);
        if (a0)
          bulk_load(st, ws + (((int64_t)b * p.hq + head[0]) * bp.ds_tiles_per_head + tl->cidx[e][0]) * 8192, 8192,
                    &tl->full[s]);
        if (a1)
          bulk_load(st + 8192, ws + (((int64_t)b * p.hq + head[1]) * bp.ds_tiles_per_head + tl->cidx[e][1]) * 8192,
                    8192, &tl->full[s]);
      }
      __syncwarp();
    }
  } else if (n > 0 && warp == kDqsIssuer) {
    // ------------------------------------------------------------ dQ += dS K
    // A = the two dS^T tiles, MN-major and un-swizzled: sixteen slabs of 8 q columns, 1 KB apart,
    // each a column of core matrices (8 kv rows x 16 bytes, 128 bytes apart); a k-step is 16 kv rows
    // = 256 bytes down every slab.  B = K read MN-major from its swizzled TMA tile (16 kv rows = 2 KB
    // per k-step, 64-dim halves 8 KB apart).
    const uint32_t idesc = umma_idesc(BF16, 128, D, true, true);
    const uint64_t adesc0 = umma_desc_plain(smem_u32(smem), 128, 1024);
    const uint64_t bdesc0 = umma_desc_sw128(smem_u32(smem) + 16384, 8192, 1024);
    bool ok = true;
    for (int e = 0; e < n && ok; ++e) {
      const int s = e % kDqsStages;
      if (!mbar_wait(&tl->full[s], (e / kDqsStages) & 1, wait_status, 332)) { ok = false; break; }
      tc_fence_after();
      const uint64_t so = (uint64_t)((s * kStageBytes) >> 4);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_ss(tmem, adesc0 + so + (uint64_t)((kk * 256) >> 4), bdesc0 + so + (uint64_t)((kk * 2048) >> 4),
                    idesc, (e | kk) ? 1u : 0u);
        tc_commit(&tl->empty[s]);
      }
      __syncwarp();
    }
    if (ok && elect_one()) tc_commit(&tl->all_done);
    __syncwarp();
  } else if (warp < 4) {
    // ------------------------------------------------------------ epilogue (or zero rows)
    const int r = tid, t = r >> 6;
    const int q_row = qblk[t] * kBS + (r & 63);
    const bool row_ok = valid[t] && q_row < p.sq && BSA_IN_BOUNDS(q_row >= 0 && head[t] < p.hq && b < p.batch, wait_status, 817);
    uint8_t* grow = reinterpret_cast<uint8_t*>(bp.dq) +
                    ((int64_t)b * bp.dq_sb + (int64_t)head[t] * bp.dq_sh + (int64_t)q_row * bp.dq_ss) * 2;
    if (n == 0) {
      if (row_ok)
        for (int i = 0; i < p.d / 4; ++i) reinterpret_cast<uint2*>(grow)[i] = make_uint2(0u, 0u);
    } else if (mbar_wait(&tl->all_done, 0, wait_status, 333)) {
      tc_fence_after();
      const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
      const bool wide = reinterpret_cast<uintptr_t>(bp.dq) % 16 == 0 && bp.dq_sb % 8 == 0 &&
                        bp.dq_sh % 8 == 0 && bp.dq_ss % 8 == 0;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_off + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * p.sm_scale, __uint_as_float(o[2 * i + 1]) * p.sm_scale);
        if (row_ok) {
          if (wide) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (ch * 32 + i * 8 < p.d)   // columns at or past the real head dim are padding
                *reinterpret_cast<uint4*>(grow + ch * 64 + i * 16) =
                    make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (ch * 32 + i * 4 < p.d)
                *reinterpret_cast<uint2*>(grow + ch * 64 + i * 8) = make_uint2(w[2 * i], w[2 * i + 1]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kDqsIssuer) tmem_dealloc(tmem, D);
}

bool rows8(const void* ptr, int64_t ss, int64_t sh, int64_t sb) {
  return reinterpret_cast<uintptr_t>(ptr) % 8 == 0 && ss % 4 == 0 && sh % 4 == 0 && sb % 4 == 0;
}

template <bool BF16, int D>
int launch_bwd(const bsa_bwd_params* bp, cudaStream_t s) {
  constexpr int kD = D;
  constexpr size_t kDkdvSmem = dkdv_smem<D>(), kDqSmem = dq_smem<D>();
  const bsa_fwd_params* p = &bp->f;
  Tmap4 tmQ, tmK, tmV, tmDO;
  // the maps carry the real head dim: columns between it and the kernels' width D come back as zeros
  (void)kD;
  int rc = make_tmap_4d(&tmQ, p->q, 2, p->d, p->sq, p->hq, p->batch, p->q_ss * 2, p->q_sh * 2, p->q_sb * 2,
                        64, 64, true, BF16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmDO, bp->d_o, 2, p->d, p->sq, p->hq, p->batch, bp->do_ss * 2, bp->do_sh * 2,
                    bp->do_sb * 2, 64, 64, true, BF16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmK, p->k, 2, p->d, p->sk, p->hkv, p->batch, p->k_ss * 2, p->k_sh * 2, p->k_sb * 2,
                    64, 64, true, BF16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, p->v, 2, p->d, p->sk, p->hkv, p->batch, p->v_ss * 2, p->v_sh * 2, p->v_sb * 2,
                    64, 64, true, BF16);
  if (rc) return rc;
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  {
    const long long rows = (long long)p->batch * p->hq * padded_sq(p->sq);
    bwd_delta_vec_kernel<BF16, D><<<(unsigned)((rows + 31) / 32), 256, 0, s>>>(*bp);
    rc = check_launch("bwd_delta_vec_kernel");
    if (rc) return rc;
  }
  {
    auto kern = bwd_dkdv_sm100_kernel<BF16, D>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDkdvSmem));
    dim3 grid(bp->kv_pairs ? bp->n_pairs : cdiv_i(cdiv_i(p->sk, kBS), 2), p->hkv, p->batch);
    kern<<<grid, kDkdvThreads, kDkdvSmem, s>>>(tmQ, tmK, tmV, tmDO, *bp, status);
    rc = check_launch("bwd_dkdv_sm100_kernel");
    if (rc) return rc;
  }
  const int G = p->hq / p->hkv;
  // as in the forward: two q heads share a tile only when they share a block list
  const int mode = (G % 2 == 0 && p->h_pat != p->hq) ? kPairHeads : kPairRows;
  if (bp->ds_ws) {
    // dQ from the dS tiles the dK/dV kernel has stored (one product per block)
    constexpr size_t kDqsSmem = dqs_smem<D>();
    auto kern = bwd_dq_from_ds_kernel<BF16, D>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqsSmem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cdiv_i(p->sq, mode == kPairHeads ? 64 : 128), mode == kPairHeads ? p->hq / 2 : p->hq,
                       p->batch);
    cfg.blockDim = dim3(kDqsThreads);
    cfg.dynamicSmemBytes = kDqsSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BSA_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tmK, *bp, mode, status));
    rc = check_launch("bwd_dq_from_ds_kernel");
  } else {
    auto kern = bwd_dq_sm100_kernel<BF16, D>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem));
    dim3 grid(cdiv_i(p->sq, mode == kPairHeads ? 64 : 128), mode == kPairHeads ? p->hq / 2 : p->hq,
              p->batch);
    // programmatic dependent of the dK/dV kernel (see the kernels' first lines)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = kDqSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BSA_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tmQ, tmK, tmV, tmDO, *bp, mode, status));
    rc = check_launch("bwd_dq_sm100_kernel");
  }
  return rc;
}

}  // namespace

bool sm100_bwd_supported(const bsa_bwd_params* bp, const char** why) {
  const bsa_fwd_params* p = &bp->f;
  auto no = [&](const char* w) { *why = w; return false; };
  if (!(p->dtype == BSA_F16 || p->dtype == BSA_BF16)) return no("dtype is not f16/bf16");
  if (p->d < 16 || p->d > 128 || p->d % 8) return no("head dim is not a multiple of 8 in [16, 128]");
  if (p->block_size != kBS) return no("block size is not 64");
  if (p->fine_block != 0 && !((p->fine_block == 16 || p->fine_block == 32) && p->col_bits && bp->ds_ws))
    return no("a fine-block pattern needs col_bits and the dS workspace");
  if (p->sk > kMaxBlocks * kBS || p->sq > kMaxBlocks * kBS) return no("more than 65536 positions");
  if ((p->hq / p->hkv) * cdiv_i(p->sq, kBS) > kMaxEntries)
    return no("group size x q blocks exceeds the per-CTA list capacity");
  if (p->hq / p->hkv > 255) return no("group size above 255");
  if (p->q_start || p->k_start || p->row_mode != BSA_ROWS_BY_TILE) return no("padded or packed batch");
  if (!tma_compatible(p->q, 2, p->q_ss, p->q_sh, p->q_sb) ||
      !tma_compatible(p->k, 2, p->k_ss, p->k_sh, p->k_sb) ||
      !tma_compatible(p->v, 2, p->v_ss, p->v_sh, p->v_sb) ||
      !tma_compatible(bp->d_o, 2, bp->do_ss, bp->do_sh, bp->do_sb))
    return no("q/k/v/dO need 16-byte aligned bases and strides that are multiples of 16 bytes");
  if (!rows8(p->o, p->o_ss, p->o_sh, p->o_sb) || !rows8(bp->d_o, bp->do_ss, bp->do_sh, bp->do_sb) ||
      !rows8(bp->dq, bp->dq_ss, bp->dq_sh, bp->dq_sb) || !rows8(bp->dk, bp->dk_ss, bp->dk_sh, bp->dk_sb) ||
      !rows8(bp->dv, bp->dv_ss, bp->dv_sh, bp->dv_sb))
    return no("o/dO/dQ/dK/dV rows are not 8-byte aligned");
  if (p->sq == 0 || p->sk == 0 || p->batch == 0) return no("empty problem");
  if (!(p->sm_scale > 0.f)) return no("sm_scale is not positive");
  return true;
}

int sm100_bwd(const bsa_bwd_params* bp, cudaStream_t s) {
  const bool bf16 = bp->f.dtype == BSA_BF16;
  // two kernel widths; a narrower head is padded with the zeros TMA supplies for out-of-range columns
  if (bp->f.d > 64) return bf16 ? launch_bwd<true, 128>(bp, s) : launch_bwd<false, 128>(bp, s);
  return bf16 ? launch_bwd<true, 64>(bp, s) : launch_bwd<false, 64>(bp, s);
}

}  // namespace bsa
