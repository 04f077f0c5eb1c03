// Bandwidth-bound decode: one query token per sequence against contiguous K/V.
//
// Grid = (split, kv head x head group, sequence).  A CTA owns up to
// blocks_per_split attended blocks of one (sequence, kv head): a producer warp
// streams their K and V tiles (64 tokens x D, 128-byte-swizzled TMA boxes) through
// a 2-stage shared-memory ring (three CTAs fit per SM, so one CTA's prologue and epilogue
// are covered by the loads of the other two), and four consumer warps each take 16 tokens of
// every tile.  The q heads of the kv group are stacked into the 16 rows of an
// m16n8k16 tensor-core tile, so K/V are read from HBM once per group, and the
// per-token work is a handful of ldmatrix + mma instructions, which keeps the
// kernel on the memory roofline.  Each warp keeps its own online-softmax state;
// warps are merged through shared memory at the end and the CTA writes either
// the final (O, LSE) (one split) or an fp32 partial that merge_kernel combines.
//
// Semantics follow the q_len == 1 case of
// dkernel/ops/sparse_attn_inference.py:503-514: positions are re-based to the
// first real token, the pattern row is (len - 1) / block_size, every real token
// of an attended block is visible.
#include <mutex>
#include <type_traits>

#include "ptx.cuh"

namespace bsa {

// Status block of the bounded waits: [0] code of the first wait that gave up (0 = none),
// [2..3] device-visible address of the host's mirror word (or null).
__device__ __align__(16) int g_wait_status[4] = {0, 0, 0, 0};

namespace {

constexpr int kStages = 2;               // K/V ring depth
constexpr int kMinCtas = 3;              // resident CTAs per SM the kernel is built for
constexpr int kTok = 64;                 // tokens per pipeline stage
constexpr int kConsumers = 4;            // consumer warps
constexpr int kDecThreads = 32 * (kConsumers + 1);
constexpr int kMaxUnits = 64;            // stage-units per CTA

template <typename T> struct MmaType;
template <> struct MmaType<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

struct DecodeSmem {
  // after the 1024-aligned stage ring
  uint64_t full[2 * kStages];   // the 8-bit K/V ring is twice as deep
  uint64_t empty[2 * kStages];
  int n_units;              // stage-units of this CTA
  int unit_pos[kMaxUnits];  // first position of each stage-unit
  float wm[kConsumers][16];
  float wl[kConsumers][16];
};

// byte offset of 16-byte chunk `chunk` (0 .. D/8-1) of token row `tok` in a tile
// stored as D/64 sub-tiles of [64 tokens][128 bytes], 128-byte swizzled
__device__ __forceinline__ uint32_t tile_off(int tok, int chunk) {
  return (uint32_t)((chunk >> 3) * (kTok * 128) + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4));
}

// Shared-memory geometry.  16-bit K/V: a stage holds a K and a V tile as the tensor cores read
// them (D/64 sub-tiles of [64 tokens][128 bytes], 128-byte swizzled).  8-bit (e4m3) K/V: a stage
// holds the two tiles as stored ([64 tokens][D bytes], half the bytes, so twice the stages keep
// the same number of bytes in flight); the consumer warps read the stored bytes with plain
// 16-byte loads and convert them straight into tensor-core fragments in registers.  e4m3 converts
// to f16 exactly and in one instruction per pair, so with an 8-bit cache the products run in f16
// whatever the type of q (q is converted once while it is staged; P lies in [0, 1]).
//
// Fragment trick of the 8-bit path: a product's contraction index may be enumerated in any order,
// and so may the output columns, as long as both operands (resp. the epilogue) agree.
//   Q K^T: thread (g, tq) of an m16n8k16 step holds k slots {2tq, 2tq+1, 8+2tq, 9+2tq}.  Over the
//          four steps of a 64-dim chunk these are made to stand for dims 16 tq .. 16 tq + 15 of the
//          chunk (step kk: dims 16 tq + 4 kk + {0,1} and + {2,3}), so a thread's share of a K row
//          is ONE 16-byte load and each of its four words converts into one step's B fragment.
//   P V:   output column j of n-tile nt stands for dim (D/8) j + nt, so thread g owns D/8
//          consecutive dims: its share of a V row is one 16-byte (D = 128) load, and a byte
//          permute pairs the bytes of two token rows into the B fragment of an n-tile.
template <int D, bool FP8> struct DecGeo {
  static constexpr int kStages = FP8 ? 2 * bsa::kStages : bsa::kStages;
  static constexpr int kTileBytes = kTok * D * (FP8 ? 1 : 2);
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kRing = kStages * kStageBytes;
  static constexpr size_t kSmem = 1024 + kRing + 16 * D * 2 + sizeof(DecodeSmem);
};

// four e4m3 bytes of a word -> two f16x2: (byte 0, byte 1) and (byte 2, byte 3); exact
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi) : "r"(w));
}
__device__ __forceinline__ uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

template <typename T, int D, bool FP8>
__global__ void __launch_bounds__(kDecThreads, kMinCtas)
decode_kernel(const __grid_constant__ Tmap4 tmK, const __grid_constant__ Tmap4 tmV,
              bsa_decode_params p, int nsplit, int* wait_status) {
  using Geo = DecGeo<D, FP8>;
  constexpr int kStages = Geo::kStages;
  constexpr int kTileBytes = Geo::kTileBytes;
  constexpr int kStageBytes = Geo::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* ring = smem;
  using MT = typename std::conditional<FP8, __half, T>::type;   // type of the tensor-core products
  MT* Qs = reinterpret_cast<MT*>(smem + Geo::kRing);  // [16][D]
  DecodeSmem* sm = reinterpret_cast<DecodeSmem*>(smem + Geo::kRing + 16 * D * 2);

  // the merge kernel behind this one may be made resident as soon as every CTA got here
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (*reinterpret_cast<volatile int*>(wait_status) != 0) return;  // an earlier wait gave up
  const int sp = blockIdx.x, b = blockIdx.z;
  const int G = p.hq / p.hkv;
  const int GH = p.heads_per_cta;
  const int groups_per_kv = G / GH;
  const int kvh = blockIdx.y / groups_per_kv;
  const int h0 = kvh * G + (blockIdx.y % groups_per_kv) * GH;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bs = p.block_size;
  const bool q_vec = reinterpret_cast<uintptr_t>(p.q) % 16 == 0 && p.q_sb % 8 == 0 && p.q_sh % 8 == 0;

  const int ks = p.k_start ? p.k_start[b] : 0;
  const int ke = p.k_end ? p.k_end[b] : p.sk;
  const int local_len = ke - ks;
  const int pos0 = p.k_pos0 ? p.k_pos0[b] : 0;
  const int total = p.k_total ? p.k_total[b] : pos0 + local_len;
  const int end_pos = p.k_blk_mod > 1 ? total : min(total, pos0 + local_len);

  // A KV shard is either a contiguous position range [pos0, pos0 + stored) or, with k_blk_mod = W
  // > 1, the blocks whose index is congruent to k_blk_rem modulo W, stored back to back (block c
  // of the sequence is local block c / W).
  const int mod = p.k_blk_mod > 1 ? p.k_blk_mod : 1;
  auto issue_unit = [&](int u) {
    const int s = u % kStages;
    mbar_expect_tx(&sm->full[s], kStageBytes);
    const int upos = sm->unit_pos[u];
    const int tok = mod == 1 ? ks + (upos - pos0) : ks + (upos / bs / mod) * bs + upos % bs;
    // a unit starts inside the stored tokens of its kv head (its tail may be past them)
    (void)BSA_IN_BOUNDS(tok >= 0 && tok < p.sk && kvh >= 0 && kvh < p.hkv && b < p.batch, wait_status, 821);
    uint8_t* kdst = ring + s * kStageBytes;
    uint8_t* vdst = kdst + kTileBytes;
    if (FP8) {   // one box of [64 tokens][D bytes] per tensor, as stored
      tma_load_tile(kdst, &tmK, &sm->full[s], 0, tok, kvh, b);
      tma_load_tile(vdst, &tmV, &sm->full[s], 0, tok, kvh, b);
    } else {
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_tile(kdst + c * (kTok * 128), &tmK, &sm->full[s], c * 64, tok, kvh, b);
        tma_load_tile(vdst + c * (kTok * 128), &tmV, &sm->full[s], c * 64, tok, kvh, b);
      }
    }
  };

  if (warp == kConsumers) {
    // ---- the producer warp finds the attended blocks of this CTA: the sp-th group of
    // blocks_per_split row entries that lie in the shard.  The row is read 32 entries at a time
    // (one coalesced load and one vote per chunk instead of a chain of dependent loads), and the
    // first tiles are requested before the rest of the CTA has staged Q.
    int nu = 0;
    if (total > 0 && local_len > 0) {
      const int row = (total - 1) / bs;
      const int hp = pattern_head(h0, p.h_pat, p.hq, p.hkv);
      int c_beg = 0, c_end = 0;
      if (row < p.n_rows) {
        const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
        c_beg = __ldg(cr + row);
        c_end = __ldg(cr + row + 1);
      }
      const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
      const int subs = bs / kTok;
      const int want0 = sp * p.blocks_per_split, want1 = want0 + p.blocks_per_split;
      int seen = 0;   // row entries of the shard met so far
      for (int e0 = c_beg; e0 < c_end && seen < want1; e0 += 32) {
        const int e = e0 + lane;
        const int c = e < c_end ? __ldg(cols + e) : -1;
        const bool mine = c >= 0 && (mod == 1 ? c * bs >= pos0 : c % mod == p.k_blk_rem);
        const uint32_t vote = __ballot_sync(0xffffffffu, mine);
        const int idx = seen + __popc(vote & ((1u << lane) - 1u));
        int valid_units = 0;
        if (mine && idx >= want0 && idx < want1) {
          for (int s = 0; s < subs; ++s) {
            // positions grow with the entry index, so the units past the end form a tail
            const int pos = c * bs + s * kTok;
            const int u = (idx - want0) * subs + s;
            if (pos < end_pos && u < kMaxUnits) {
              sm->unit_pos[u] = pos;
              ++valid_units;
            }
          }
        }
        nu += __reduce_add_sync(0xffffffffu, valid_units);
        seen += __popc(vote);
      }
    }
    __syncwarp();
    if (lane == 0) {
      sm->n_units = nu;
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&sm->full[s], 1);
        mbar_init(&sm->empty[s], kConsumers);
      }
      mbar_fence_init();
      for (int u = 0; u < nu && u < kStages; ++u) issue_unit(u);
    }
  } else {
    // q heads of the group -> rows of the 16-row A tile (rows >= GH are zero), 16 bytes a thread
    for (int i = tid; i < 16 * D / 8; i += kConsumers * 32) {
      const int r = i / (D / 8), c = i % (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < GH) {
        const T* src = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)(h0 + r) * p.q_sh + c * 8;
        if (q_vec) {
          v = *reinterpret_cast<const uint4*>(src);
        } else {
          T tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) tmp[e] = src[e];
          v = *reinterpret_cast<const uint4*>(tmp);
        }
        if (!std::is_same<MT, T>::value) {   // bf16 queries against an 8-bit cache: products run in f16
          const T* e = reinterpret_cast<const T*>(&v);
          __half hq[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) hq[j] = __float2half_rn(fminf(fmaxf(Elem<T>::to_f(e[j]), -65504.f), 65504.f));
          v = *reinterpret_cast<const uint4*>(hq);
        }
      }
      reinterpret_cast<uint4*>(Qs)[i] = v;
    }
  }
  __syncthreads();
  const int n_units = sm->n_units;
  // one split and an output tensor: write the final rows; otherwise an fp32 partial per split
  const bool final_out = nsplit == 1 && p.o != nullptr;

  if (n_units == 0) {  // nothing attended here: an empty partial (uniform exit)
    for (int i = tid; i < GH * D; i += kDecThreads) {
      const int h = h0 + i / D, d = i % D;
      if (final_out) {
        reinterpret_cast<T*>(p.o)[(int64_t)b * p.o_sb + (int64_t)h * p.o_sh + d] = Elem<T>::from_f(0.f);
      } else {
        p.ws[(((int64_t)b * p.hq + h) * nsplit + sp) * D + d] = 0.f;
      }
    }
    for (int i = tid; i < GH; i += kDecThreads) {
      const int h = h0 + i;
      if (final_out) {
        if (p.lse) p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh] = -INFINITY;
      } else {
        p.ws[(int64_t)p.batch * p.hq * nsplit * D + ((int64_t)b * p.hq + h) * nsplit + sp] = -INFINITY;
      }
    }
    return;
  }

  const int g = lane >> 2, tq = lane & 3;
  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

  if (warp == kConsumers) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      for (int u = kStages; u < n_units; ++u) {   // the first kStages units are already in flight
        const int s = u % kStages;
        const uint32_t ph = (u / kStages) & 1;
        if (!mbar_wait(&sm->empty[s], ph ^ 1, wait_status, 101)) break;
        issue_unit(u);
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t* q32 = reinterpret_cast<const uint32_t*>(Qs);
      // k slots (2tq, 2tq+1) and (8+2tq, 9+2tq) of step kk: the dims of the same numbers, or
      // (8-bit K/V) dims 16 tq + 4 (kk % 4) + {0,1} / {2,3} of 64-dim chunk kk / 4
      const int d0 = FP8 ? (kk >> 2) * 64 + tq * 16 + (kk & 3) * 4 : kk * 16 + tq * 2;
      const int d1 = FP8 ? d0 + 2 : d0 + 8;
      qa[kk][0] = q32[(g * D + d0) >> 1];
      qa[kk][1] = q32[((g + 8) * D + d0) >> 1];
      qa[kk][2] = q32[(g * D + d1) >> 1];
      qa[kk][3] = q32[((g + 8) * D + d1) >> 1];
    }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    // e4m3 K carries a per-tensor scale: it folds into the logit scale (V's goes on the output)
    const float scale2 = p.sm_scale * kLog2e * (FP8 ? p.k_scale : 1.f);
    const uint32_t ring_u32 = smem_u32(ring);
    bool alive = true;

    for (int u = 0; u < n_units && alive; ++u) {
      const int s = u % kStages;
      const uint32_t ph = (u / kStages) & 1;
      alive = mbar_wait(&sm->full[s], ph, wait_status, 102);
      if (!alive) break;
      const int pos_u = sm->unit_pos[u];
      const uint32_t kbase = ring_u32 + s * kStageBytes;
      const uint32_t vbase = kbase + kTileBytes;
      const int valid = end_pos - pos_u;  // tokens of this unit that exist (may exceed 64)
      const uint8_t* k8 = ring + s * kStageBytes;    // the tiles as generic pointers (8-bit path)
      const uint8_t* v8 = k8 + kTileBytes;
      if (FP8) {
        // nothing to prepare: rows past the end of the sequence are zeroed when V is read
      } else if (valid < kTok) {
        // rows past the end of the sequence may hold anything: clear them in V so
        // that 0 * garbage cannot produce NaN
        uint8_t* vgen = ring + s * kStageBytes + kTileBytes;
        for (int t = warp * 16; t < warp * 16 + 16; ++t) {
          if (t >= valid) {
#pragma unroll
            for (int c = 0; c < D / 64; ++c)
              reinterpret_cast<uint32_t*>(vgen + c * (kTok * 128) + t * 128)[lane] = 0u;
          }
        }
        fence_proxy_async();  // order these writes before the next TMA into the stage
        __syncwarp();
      }
      // S = Q K^T for this warp's 16 tokens
      float sacc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
        if (FP8) {
          const int tok = warp * 16 + nt * 8 + g;      // B fragment column n = g
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            const uint4 kb = *reinterpret_cast<const uint4*>(k8 + tok * D + c * 64 + tq * 16);
            const uint32_t w[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              uint32_t b0, b1;
              cvt_e4m3x4(w[kk], b0, b1);
              MmaType<MT>::mma(sacc[nt], qa[c * 4 + kk], b0, b1);
            }
          }
        } else {
          const int tok = warp * 16 + nt * 8 + (lane & 7);
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk) {
            uint32_t r0, r1, r2, r3;
            ldsm_x4(kbase + tile_off(tok, kk * 4 + (lane >> 3)), r0, r1, r2, r3);
            MmaType<MT>::mma(sacc[nt], qa[2 * kk], r0, r1);
            MmaType<MT>::mma(sacc[nt], qa[2 * kk + 1], r2, r3);
          }
        }
      }
      // mask + online softmax (rows g and g+8)
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = warp * 16 + nt * 8 + tq * 2 + e;
          const bool ok = t < valid;
          sacc[nt][e] = ok ? sacc[nt][e] * scale2 : -INFINITY;
          sacc[nt][2 + e] = ok ? sacc[nt][2 + e] * scale2 : -INFINITY;
          mx_lo = fmaxf(mx_lo, sacc[nt][e]);
          mx_hi = fmaxf(mx_hi, sacc[nt][2 + e]);
        }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo;
      const float ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float a_lo = exp2f(m_lo - ms_lo), a_hi = exp2f(m_hi - ms_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      uint32_t pa[4];
      {
        const float p00 = exp2f(sacc[0][0] - ms_lo), p01 = exp2f(sacc[0][1] - ms_lo);
        const float p02 = exp2f(sacc[0][2] - ms_hi), p03 = exp2f(sacc[0][3] - ms_hi);
        const float p10 = exp2f(sacc[1][0] - ms_lo), p11 = exp2f(sacc[1][1] - ms_lo);
        const float p12 = exp2f(sacc[1][2] - ms_hi), p13 = exp2f(sacc[1][3] - ms_hi);
        l_lo = l_lo * a_lo + (p00 + p01 + p10 + p11);
        l_hi = l_hi * a_hi + (p02 + p03 + p12 + p13);
        pa[0] = MmaType<MT>::pack(p00, p01);
        pa[1] = MmaType<MT>::pack(p02, p03);
        pa[2] = MmaType<MT>::pack(p10, p11);
        pa[3] = MmaType<MT>::pack(p12, p13);
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        oacc[i][0] *= a_lo; oacc[i][1] *= a_lo;
        oacc[i][2] *= a_hi; oacc[i][3] *= a_hi;
      }
      // O += P V over this warp's 16 tokens
      if (FP8) {
        // k slots (2tq, 2tq+1, 8+2tq, 9+2tq) are this warp's token rows of the same numbers; the
        // thread's D/8 consecutive dims of each row arrive in one load (zero past the sequence end)
        constexpr int kNT = D / 8;                       // n-tiles = dims per thread
        uint32_t rows[4][kNT / 4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = warp * 16 + (i >> 1) * 8 + tq * 2 + (i & 1);
          const uint8_t* src = v8 + tok * D + g * kNT;
          if (kNT == 16) {
            const uint4 r = tok < valid ? *reinterpret_cast<const uint4*>(src) : make_uint4(0u, 0u, 0u, 0u);
            rows[i][0] = r.x; rows[i][1] = r.y; rows[i][kNT / 4 - 2] = r.z; rows[i][kNT / 4 - 1] = r.w;
          } else {
            const uint2 r = tok < valid ? *reinterpret_cast<const uint2*>(src) : make_uint2(0u, 0u);
            rows[i][0] = r.x; rows[i][kNT / 4 - 1] = r.y;
          }
        }
#pragma unroll
        for (int nt2 = 0; nt2 < kNT / 2; ++nt2) {         // two n-tiles (dims 2 nt2, 2 nt2 + 1 of the thread) per permute
          const int wi = nt2 >> 1;
          const uint32_t sel = (nt2 & 1) ? 0x7362u : 0x5140u;   // {a.b, b.b, a.b+1, b.b+1}, b = 0 or 2
          uint32_t b0a, b0b, b1a, b1b;
          cvt_e4m3x4(byte_perm(rows[0][wi], rows[1][wi], sel), b0a, b0b);   // tokens 2tq, 2tq+1
          cvt_e4m3x4(byte_perm(rows[2][wi], rows[3][wi], sel), b1a, b1b);   // tokens 8+2tq, 9+2tq
          MmaType<MT>::mma(oacc[2 * nt2], pa, b0a, b1a);
          MmaType<MT>::mma(oacc[2 * nt2 + 1], pa, b0b, b1b);
        }
      } else {
#pragma unroll
        for (int dn = 0; dn < D / 16; ++dn) {
          const int mi = lane >> 3;
          const int tok = warp * 16 + (mi & 1) * 8 + (lane & 7);
          uint32_t r0, r1, r2, r3;
          ldsm_x4_t(vbase + tile_off(tok, dn * 2 + (mi >> 1)), r0, r1, r2, r3);
          MmaType<MT>::mma(oacc[2 * dn], pa, r0, r1);
          MmaType<MT>::mma(oacc[2 * dn + 1], pa, r2, r3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->empty[s]);
    }
    // quad-reduce the row sums
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (tq == 0) {
      sm->wm[warp][g] = m_lo; sm->wm[warp][g + 8] = m_hi;
      sm->wl[warp][g] = l_lo; sm->wl[warp][g + 8] = l_hi;
    }
  }
  __syncthreads();  // every tile has been consumed: the ring is free
  if (warp < kConsumers) {
    float* Omw = reinterpret_cast<float*>(ring);  // [kConsumers][16][D]
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      // column j = 2tq (+1) of n-tile i is dim 8 i + j, or (8-bit K/V) dim (D/8) j + i
      const int d0 = FP8 ? (D / 8) * (tq * 2) + i : i * 8 + tq * 2;
      const int d1 = FP8 ? d0 + D / 8 : d0 + 1;
      float* lo = Omw + ((warp * 16 + g) * D);
      float* hi = Omw + ((warp * 16 + g + 8) * D);
      lo[d0] = oacc[i][0]; lo[d1] = oacc[i][1];
      hi[d0] = oacc[i][2]; hi[d1] = oacc[i][3];
    }
  }
  __syncthreads();  // partial outputs are in shared memory

  const float* Om = reinterpret_cast<const float*>(ring);
  for (int i = tid; i < GH * D; i += kDecThreads) {
    const int r = i / D, d = i % D;
    float mf = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumers; ++w) mf = fmaxf(mf, sm->wm[w][r]);
    const float msafe = mf == -INFINITY ? 0.f : mf;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumers; ++w) {
      const float sc = exp2f(sm->wm[w][r] - msafe);
      acc += Om[(w * 16 + r) * D + d] * sc;
      l += sm->wl[w][r] * sc;
    }
    const float inv = (l > 0.f ? 1.f / l : 0.f) * (FP8 ? p.v_scale : 1.f);   // e4m3 V: per-tensor scale
    const float lse = l > 0.f ? (mf + log2f(l)) * kLn2 : -INFINITY;
    const int h = h0 + r;
    if (final_out) {
      reinterpret_cast<T*>(p.o)[(int64_t)b * p.o_sb + (int64_t)h * p.o_sh + d] =
          Elem<T>::from_f(acc * inv);
      if (d == 0 && p.lse) p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh] = lse;
    } else {
      if (BSA_IN_BOUNDS(h < p.hq && sp < nsplit && d < D, wait_status, 822))
        p.ws[(((int64_t)b * p.hq + h) * nsplit + sp) * D + d] = acc * inv;
      if (d == 0)
        p.ws[(int64_t)p.batch * p.hq * nsplit * D + ((int64_t)b * p.hq + h) * nsplit + sp] = lse;
    }
  }
}

// out[row] = sum_p o_p[row] * softmax_p(lse_p[row]); merged lse = logsumexp_p.
template <typename Tin, typename Tout>
__global__ void merge_kernel(const Tin* __restrict__ o_parts, const float* __restrict__ lse_parts,
                             int P, int64_t rows, int d, int64_t pso, int64_t rso, int64_t psl,
                             int64_t rsl, Tout* __restrict__ o, int64_t ors,
                             float* __restrict__ lse, int64_t lrs) {
  const int64_t total = rows * d;
  // Launched as a programmatic dependent of the decode kernel: the blocks may already be
  // resident while that grid drains, and wait here until its partials are visible.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / d;
    const int c = (int)(i - r * d);
    float mx = -INFINITY;
    for (int q = 0; q < P; ++q) mx = fmaxf(mx, lse_parts[q * psl + r * rsl]);
    const float ms = mx == -INFINITY ? 0.f : mx;
    float den = 0.f, acc = 0.f;
    for (int q = 0; q < P; ++q) {
      const float w = __expf(lse_parts[q * psl + r * rsl] - ms);
      den += w;
      if (w != 0.f) acc += w * Elem<Tin>::to_f(o_parts[q * pso + r * rso + c]);
    }
    o[r * ors + c] = Elem<Tout>::from_f(den > 0.f ? acc / den : 0.f);
    if (c == 0 && lse) lse[r * lrs] = den > 0.f ? ms + __logf(den) : -INFINITY;
  }
}

template <typename Tin, typename Tout>
int launch_merge(const void* o_parts, const float* lse_parts, int P, int64_t rows, int d,
                 int64_t pso, int64_t rso, int64_t psl, int64_t rsl, void* o, int64_t ors,
                 float* lse, cudaStream_t s, int64_t lrs = 1) {
  const int64_t total = rows * d;
  if (total == 0) return BSA_OK;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  BSA_CHECK_CUDA(cudaLaunchKernelEx(&cfg, merge_kernel<Tin, Tout>, reinterpret_cast<const Tin*>(o_parts),
                                    lse_parts, P, rows, d, pso, rso, psl, rsl,
                                    reinterpret_cast<Tout*>(o), ors, lse, lrs));
  return check_launch("merge_kernel");
}

// Checks that must hold before any arithmetic on the head counts (the split planning divides by
// them): shared by bsa_decode, bsa_decode_static and bsa_decode_workspace_bytes.
int decode_validate_heads(const bsa_decode_params* p, const char* who) {
  BSA_CHECK_ARG(p, "%s: null params", who);
  BSA_CHECK_ARG(p->batch >= 0 && p->hq >= 1 && p->hkv >= 1 && p->hq % p->hkv == 0,
                "%s: bad head counts hq=%d hkv=%d", who, p->hq, p->hkv);
  const int G = p->hq / p->hkv;
  BSA_CHECK_ARG(p->heads_per_cta >= 1 && p->heads_per_cta <= 16 && G % p->heads_per_cta == 0,
                "%s: heads_per_cta=%d must divide the group size %d and be <= 16", who,
                p->heads_per_cta, G);
  BSA_CHECK_ARG(p->d >= 1 && p->max_row_nnz >= 0, "%s: bad sizes d=%d max_row_nnz=%d", who, p->d,
                p->max_row_nnz);
  BSA_CHECK_ARG(p->k_blk_mod >= 0 && (p->k_blk_mod <= 1 || (p->k_blk_rem >= 0 && p->k_blk_rem < p->k_blk_mod)),
                "%s: bad block-cyclic shard %d mod %d", who, p->k_blk_rem, p->k_blk_mod);
  return BSA_OK;
}

// Attended blocks per CTA.  A caller's choice is kept; otherwise a CTA gets as many blocks as
// possible (up to 16: one prologue and one partial per 512 KB of K/V) while the grid still
// fills the machine about twice over (three resident CTAs per SM).
int decode_blocks_per_split(const bsa_decode_params* p) {
  if (p->blocks_per_split > 0) return p->blocks_per_split;
  const int hpc = p->heads_per_cta > 0 ? p->heads_per_cta : 1;
  const long long items = (long long)p->batch * p->hkv * ((p->hq / p->hkv) / hpc);
  const long long want = 2LL * 148 * kMinCtas;
  long long splits = items > 0 ? (want + items - 1) / items : 1;
  if (splits < 1) splits = 1;
  const int nnz = p->max_row_nnz > 0 ? p->max_row_nnz : 1;
  long long bps = (nnz + splits - 1) / splits;
  bps = (bps + 3) / 4 * 4;
  if (bps < 4) bps = 4;
  if (bps > 16) bps = 16;
  return (int)bps;
}

int decode_nsplit(const bsa_decode_params* p) {
  const int bps = decode_blocks_per_split(p);
  const int n = (p->max_row_nnz + bps - 1) / bps;
  return n < 1 ? 1 : n;
}

template <typename T, int D, bool FP8>
int launch_decode(const bsa_decode_params* p, cudaStream_t s) {
  Tmap4 tmK, tmV;
  const bool bf16 = p->dtype == BSA_BF16;
  const int eb = FP8 ? 1 : 2;
  const uint32_t box_d = FP8 ? D : 64;    // 8-bit tiles are copied as stored, 16-bit ones 128-byte swizzled
  int rc = make_tmap_4d(&tmK, p->k, eb, D, p->sk, p->hkv, p->batch, p->k_ss * eb, p->k_sh * eb,
                        p->k_sb * eb, box_d, kTok, !FP8, bf16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, p->v, eb, D, p->sk, p->hkv, p->batch, p->v_ss * eb, p->v_sh * eb,
                    p->v_sb * eb, box_d, kTok, !FP8, bf16);
  if (rc) return rc;
  const int nsplit = decode_nsplit(p);
  const size_t smem = DecGeo<D, FP8>::kSmem;
  auto kern = decode_kernel<T, D, FP8>;
  BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int G = p->hq / p->hkv;
  dim3 grid(nsplit, p->hkv * (G / p->heads_per_cta), p->batch);
  bsa_decode_params q = *p;
  q.blocks_per_split = decode_blocks_per_split(p);
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  kern<<<grid, kDecThreads, smem, s>>>(tmK, tmV, q, nsplit, status);
  rc = check_launch("decode_kernel");
  if (rc) return rc;
  if (nsplit > 1 && p->o) {
    const int64_t rows = (int64_t)p->batch * p->hq;
    float* ws_lse = p->ws + rows * nsplit * D;
    // partial o: (rows, nsplit, D) -> partition stride D, row stride nsplit*D
    // the merged rows are written through (o_sb, o_sh): one launch per batch row
    // layout unless o is contiguous over (batch, head)
    // rows of o and lse may be strided (e.g. packed side by side in one buffer), but batch
    // and head must collapse into one row index
    if (p->o_sb == (int64_t)p->hq * p->o_sh && (!p->lse || p->lse_sb == (int64_t)p->hq * p->lse_sh)) {
      if (bf16)
        return launch_merge<float, __nv_bfloat16>(p->ws, ws_lse, nsplit, rows, D, D,
                                                  (int64_t)nsplit * D, 1, nsplit, p->o, p->o_sh,
                                                  p->lse, s, p->lse_sh);
      return launch_merge<float, __half>(p->ws, ws_lse, nsplit, rows, D, D, (int64_t)nsplit * D, 1,
                                         nsplit, p->o, p->o_sh, p->lse, s, p->lse_sh);
    }
    set_error("bsa_decode: with several splits o and lse need batch stride = heads x head stride");
    return BSA_E_UNSUPPORTED;
  }
  return BSA_OK;
}

}  // namespace

size_t decode_workspace_bytes(const bsa_decode_params* p) {
  if (decode_validate_heads(p, "bsa_decode_workspace_bytes") != BSA_OK) return 0;
  const int nsplit = decode_nsplit(p);
  if (nsplit <= 1 && p->o) return 0;   // without an output tensor even a single split stays a partial
  return sizeof(float) * (size_t)p->batch * p->hq * nsplit * (p->d + 1);
}

int decode_run(const bsa_decode_params* p, cudaStream_t s) {
  int vrc = decode_validate_heads(p, "bsa_decode");
  if (vrc) return vrc;
  BSA_CHECK_ARG(p->q && p->k && p->v && (p->o || p->ws) && p->crow && p->col, "bsa_decode: null pointer");
  BSA_CHECK_ARG(p->h_pat == 1 || p->h_pat == p->hkv || p->h_pat == p->hq,
                "bsa_decode: pattern has %d heads, expected 1, %d or %d", p->h_pat, p->hkv, p->hq);
  if (p->batch == 0) return BSA_OK;
  if (!(p->dtype == BSA_F16 || p->dtype == BSA_BF16) || !(p->d == 64 || p->d == 128) ||
      !(p->block_size == 64 || p->block_size == 128)) {
    set_error("bsa_decode: needs f16/bf16, head dim 64 or 128 and block size 64 or 128 "
              "(got dtype %d, d %d, block %d)", p->dtype, p->d, p->block_size);
    return BSA_E_UNSUPPORTED;
  }
  const bool fp8 = p->kv_dtype == BSA_F8E4M3;
  BSA_CHECK_ARG(p->kv_dtype == 0 || fp8, "bsa_decode: kv_dtype must be 0 (as q) or BSA_F8E4M3, got %d", p->kv_dtype);
  BSA_CHECK_ARG(!fp8 || (p->k_scale > 0.f && p->v_scale > 0.f), "bsa_decode: e4m3 K/V need positive k_scale and v_scale");
  if (!tma_compatible(p->k, fp8 ? 1 : 2, p->k_ss, p->k_sh, p->k_sb) ||
      !tma_compatible(p->v, fp8 ? 1 : 2, p->v_ss, p->v_sh, p->v_sb)) {
    set_error("bsa_decode: K/V need a 16-byte aligned base and strides that are multiples of 16 bytes");
    return BSA_E_UNSUPPORTED;
  }
  const int bps = decode_blocks_per_split(p);
  if (bps * (p->block_size / kTok) > kMaxUnits) {
    set_error("bsa_decode: blocks_per_split=%d too large (limit %d tiles of 64 tokens per CTA)", bps,
              kMaxUnits);
    return BSA_E_TOOBIG;
  }
  const int nsplit = decode_nsplit(p);
  BSA_CHECK_ARG((nsplit == 1 && p->o) || p->ws, "bsa_decode: workspace required for %d splits", nsplit);
  if (fp8) {
    if (p->dtype == BSA_BF16)
      return p->d == 128 ? launch_decode<__nv_bfloat16, 128, true>(p, s) : launch_decode<__nv_bfloat16, 64, true>(p, s);
    return p->d == 128 ? launch_decode<__half, 128, true>(p, s) : launch_decode<__half, 64, true>(p, s);
  }
  if (p->dtype == BSA_BF16)
    return p->d == 128 ? launch_decode<__nv_bfloat16, 128, false>(p, s) : launch_decode<__nv_bfloat16, 64, false>(p, s);
  return p->d == 128 ? launch_decode<__half, 128, false>(p, s) : launch_decode<__half, 64, false>(p, s);
}

int merge_partials(const void* o_parts, const float* lse_parts, int P, int64_t rows, int d,
                   int64_t pso, int64_t rso, int64_t psl, int64_t rsl, void* o, int64_t ors,
                   float* lse, int dtype, cudaStream_t s) {
  BSA_CHECK_ARG(o_parts && lse_parts && o, "bsa_merge_partials: null pointer");
  BSA_CHECK_ARG(P >= 1 && rows >= 0 && d >= 1, "bsa_merge_partials: bad sizes P=%d d=%d", P, d);
  switch (dtype) {
    case BSA_F16: return launch_merge<__half, __half>(o_parts, lse_parts, P, rows, d, pso, rso, psl, rsl, o, ors, lse, s);
    case BSA_BF16: return launch_merge<__nv_bfloat16, __nv_bfloat16>(o_parts, lse_parts, P, rows, d, pso, rso, psl, rsl, o, ors, lse, s);
    case BSA_F32: return launch_merge<float, float>(o_parts, lse_parts, P, rows, d, pso, rso, psl, rsl, o, ors, lse, s);
  }
  set_error("bsa_merge_partials: unknown dtype %d", dtype);
  return BSA_E_BADARG;
}

}  // namespace bsa

namespace bsa {
// Device address of the status word of the current device (the symbol name is
// only a host-side handle; kernels get the real address as an argument).
int* wait_status_ptr() {
  static int* cache[64] = {nullptr};
  static std::mutex mu;   // entry points may be called from several host threads
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  if (!cache[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_wait_status);
    if (e != cudaSuccess) {
      set_error("cudaGetSymbolAddress(g_wait_status) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = static_cast<int*>(ptr);
  }
  return cache[dev];
}

static int* g_mirror_host[64] = {nullptr};   // the registered mirror word of each device

int read_wait_status(int* out, int reset) {
  BSA_CHECK_ARG(out, "bsa_wait_status: null pointer");
  BSA_CHECK_CUDA(cudaDeviceSynchronize());
  BSA_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_wait_status, sizeof(int)));
  if (reset && *out != 0) {
    const int zero = 0;
    BSA_CHECK_CUDA(cudaMemcpyToSymbol(g_wait_status, &zero, sizeof(int)));
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_mirror_host[dev])
      *reinterpret_cast<volatile int*>(g_mirror_host[dev]) = 0;
  }
  return BSA_OK;
}

int set_wait_status_mirror(int* host_word) {
  int dev = 0;
  BSA_CHECK_CUDA(cudaGetDevice(&dev));
  BSA_CHECK_ARG(dev >= 0 && dev < 64, "bsa_set_wait_status_mirror: device index out of range");
  int* dptr = nullptr;
  if (host_word) {
    cudaError_t e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&dptr), host_word, 0);
    if (e != cudaSuccess || !dptr) {
      (void)cudaGetLastError();
      set_error("bsa_set_wait_status_mirror: the word must be page-locked host memory that the device "
                "can address (%s)", cudaGetErrorString(e));
      return BSA_E_BADARG;
    }
  }
  BSA_CHECK_CUDA(cudaMemcpyToSymbol(g_wait_status, &dptr, sizeof(dptr), 2 * sizeof(int)));
  g_mirror_host[dev] = host_word;
  return BSA_OK;
}

// A wait that nothing will ever satisfy, with a short limit: exercises the give-up path
// (status block, mirror word, no-op behaviour of later launches) without faulting the GPU.
__global__ void wait_timeout_selftest_kernel(int* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    mbar_wait(&bar, 0, status, 900, limit_ns);   // nobody arrives
  }
}

int selftest_wait_timeout(uint32_t limit_us, cudaStream_t s) {
  BSA_CHECK_ARG(limit_us >= 1 && limit_us <= 100000, "bsa_selftest_wait_timeout: limit must be 1..100000 us");
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(status, (uint64_t)limit_us * 1000ull);
  return check_launch("wait_timeout_selftest_kernel");
}
}  // namespace bsa

// ---------------------------------------------------------------------------
// Decode without any allocation by the caller.
//
// Some hosts of this library cannot hand it scratch memory: a serving runtime
// that has pinned its whole device-memory budget to the KV cache, a plugin
// loaded into a process whose allocator it must not touch, a language binding
// that only passes through the tensors it was given.  For them the split-KV
// partials live in a fixed array that is part of the library image.  Every GPU
// that loads the library carries the array (kStaticScratchBytes) until the
// process exits.
// ---------------------------------------------------------------------------
namespace bsa {

constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of g_decode_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel can
// use, so the address is looked up once per device (with that device current)
// and handed to the kernels as an ordinary pointer.
static float* static_scratch_ptr() {
  static float* cache[64] = {nullptr};
  static std::mutex mu;   // entry points may be called from several host threads
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("bsa_decode_static: cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  if (!cache[dev]) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_decode_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("bsa_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = ptr;
  }
  return cache[dev];
}

size_t decode_static_capacity() { return kStaticScratchBytes; }

int decode_run_static(const bsa_decode_params* p, cudaStream_t s) {
  int vrc = decode_validate_heads(p, "bsa_decode_static");
  if (vrc) return vrc;
  const size_t need = decode_workspace_bytes(p);
  if (need > kStaticScratchBytes) {
    set_error("bsa_decode_static: this call needs %zu bytes of split-KV scratch but the built-in "
              "array holds %zu; lower batch*heads, raise blocks_per_split, or use bsa_decode with a "
              "caller-provided workspace", need, (size_t)kStaticScratchBytes);
    return BSA_E_TOOBIG;
  }
  float* scratch = static_scratch_ptr();
  if (!scratch) return BSA_E_CUDA;
  bsa_decode_params q = *p;
  q.ws = scratch;  // every (sequence, head, split) slot in use is rewritten by the kernel
  return decode_run(&q, s);
}

}  // namespace bsa
