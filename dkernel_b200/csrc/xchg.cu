// KV-sharded decode: exchange of the ranks' partial (O, LSE) rows and their merge, in ONE kernel
// per rank, over peer memory (NVLink) -- no library collective, no fence, no separate flag.
//
// Every rank owns an exchange buffer that all ranks of the node have mapped (CUDA IPC / symmetric
// memory; the host passes the W mapped addresses).  Data travels as 8-byte words {4 bytes of
// payload, 4 bytes = step number}: a word is written by one store and read by one load, so a
// reader that sees the current step number in a word also sees its payload, whatever the order in
// which the words of a row arrive.  Per step, on every rank r:
//   push   each thread turns 16 bytes of this rank's partial row into four such words and stores
//          them into slot r of every PEER's buffer (two 16-byte stores per destination); its own
//          copy stays in registers;
//   wait   the same thread reads the words of its 16 bytes from the peers' slots of the LOCAL
//          buffer, spinning -- bounded -- on words whose step number is not the current one,
//          merges the W partials with the semantics of combine_attn_partitions
//          (dkernel/interface.py:319-324) and writes the result.
// Only stores cross NVLink; every load is from local memory.  A thread's first action is a push and
// every wait is for words that some thread pushes before it waits for anything: the kernel
// cannot deadlock.  The step number lives in the buffer and is advanced by the last CTA to
// finish, so a captured CUDA graph can be replayed.  Slots are double buffered by step parity:
// a rank can be at most one step ahead of a peer (finishing a step needs that peer's words of the
// step), so the slot it overwrites two steps later has been consumed, and a stale word carries a
// step number that is off by two.
#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kXThreads = 256;
constexpr int kXMaxGrid = 128;      // <= SM count: every CTA is resident
constexpr int kXMaxWorld = 8;

struct XLayout {
  size_t o_off, lse_off, ctrl_off, total;
  size_t slot_o, slot_lse;   // bytes of one (parity, source rank) slot, flag words included
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ inline XLayout xlayout(int world, int64_t rows, int d) {
  XLayout L;
  L.slot_o = align_up((size_t)rows * d * 2 * 2, 256);   // every 4 payload bytes travel with 4 flag bytes
  L.slot_lse = align_up((size_t)rows * 8, 256);
  L.o_off = 0;
  L.lse_off = L.o_off + 2 * (size_t)world * L.slot_o;
  L.ctrl_off = L.lse_off + 2 * (size_t)world * L.slot_lse;
  L.total = L.ctrl_off + 256;
  return L;
}

struct XPtrs { uint8_t* buf[kXMaxWorld]; };

__device__ __forceinline__ void st_words(void* p, uint32_t a, uint32_t fa, uint32_t b, uint32_t fb) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(fa), "r"(b), "r"(fb) : "memory");
}
__device__ __forceinline__ uint4 ld_words(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_word(void* p, uint32_t a, uint32_t fa) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(fa) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kXThreads)
xchg_merge_kernel(XPtrs ptrs, int world, int rank, int64_t rows, int d, const T* __restrict__ stage_o,
                  const float* __restrict__ stage_lse, const float* __restrict__ part_o,
                  const float* __restrict__ part_lse, int nsplit, T* __restrict__ out,
                  float* __restrict__ out_lse, int* wait_status) {
  // May be launched as a programmatic dependent of the decode kernel that produces its input:
  // nothing of that kernel's output is touched before this wait (a no-op after a plain launch).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (*reinterpret_cast<volatile int*>(wait_status) != 0) return;
  const XLayout L = xlayout(world, rows, d);
  uint8_t* mine = ptrs.buf[rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(mine + L.ctrl_off);   // [0] step, [1] CTAs done
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(ctrl) + 1u;
  const int par = (int)(step & 1u);
  const int tid = threadIdx.x, cta = blockIdx.x;
  const int64_t rpc = (rows + gridDim.x - 1) / gridDim.x;
  const int64_t r0 = cta * rpc, r1 = min(rows, r0 + rpc);
  const int cpr = d / 8;                                   // 16-byte chunks per row
  const int64_t n_items = (r1 > r0 ? (r1 - r0) : 0) * cpr;
  const size_t slot_o_w = (size_t)(par * world + rank) * L.slot_o;     // where this rank writes
  const size_t slot_l_w = (size_t)(par * world + rank) * L.slot_lse;

  // ---- per 16 bytes of a row: this rank's words go to slot `rank` of every PEER's buffer (the
  // thread keeps its own copy in registers), then the same 16 bytes of every peer are awaited in
  // the local buffer.  A thread's first action is a push, so no wait can be circular.
  const uint8_t* po = mine + L.o_off + (size_t)par * world * L.slot_o;
  const uint8_t* pl = mine + L.lse_off + (size_t)par * world * L.slot_lse;
  bool failed = false;
  for (int64_t i = tid; i < n_items && !failed; i += kXThreads) {
    const int64_t r = r0 + i / cpr;
    const int c = (int)(i % cpr);
    uint4 v;
    uint32_t l;
    if (stage_o) {
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(stage_o) + (r * d + c * 8) * 2);
      l = __float_as_uint(stage_lse[r]);
    } else {
      // merge the split-KV partials of this rank first (each normalised by its own LSE)
      float mx = -INFINITY;
      for (int q = 0; q < nsplit; ++q) mx = fmaxf(mx, part_lse[r * nsplit + q]);
      const float ms = mx == -INFINITY ? 0.f : mx;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float den = 0.f;
      for (int q = 0; q < nsplit; ++q) {
        const float wt = __expf(part_lse[r * nsplit + q] - ms);
        den += wt;
        if (wt != 0.f) {
          const float4* src = reinterpret_cast<const float4*>(part_o + ((size_t)(r * nsplit + q) * d + c * 8));
          const float4 a = src[0], b2 = src[1];
          acc[0] += wt * a.x; acc[1] += wt * a.y; acc[2] += wt * a.z; acc[3] += wt * a.w;
          acc[4] += wt * b2.x; acc[5] += wt * b2.y; acc[6] += wt * b2.z; acc[7] += wt * b2.w;
        }
      }
      const float inv = den > 0.f ? 1.f / den : 0.f;
      T* e = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = Elem<T>::from_f(acc[j] * inv);
      l = __float_as_uint(den > 0.f ? ms + __logf(den) : -INFINITY);
    }
    const size_t off = ((size_t)(r * d + c * 8) * 2) * 2;
    for (int w = 0; w < world; ++w) {
      if (w == rank) continue;
      uint8_t* dst = ptrs.buf[w];
      st_words(dst + L.o_off + slot_o_w + off, v.x, step, v.y, step);
      st_words(dst + L.o_off + slot_o_w + off + 16, v.z, step, v.w, step);
      if (c == 0) st_word(dst + L.lse_off + slot_l_w + (size_t)r * 8, l, step);
    }
    uint32_t pay[kXMaxWorld][4];
    float lse_w[kXMaxWorld];
    uint32_t pending = ((1u << world) - 1u) & ~(1u << rank);
#pragma unroll
    for (int w = 0; w < kXMaxWorld; ++w) {
      if (w == rank) {
        pay[w][0] = v.x; pay[w][1] = v.y; pay[w][2] = v.z; pay[w][3] = v.w;
        lse_w[w] = __uint_as_float(l);
      }
    }
    const uint64_t t0 = global_timer_ns();
    while (pending) {
#pragma unroll
      for (int w = 0; w < kXMaxWorld; ++w) {
        if (w < world && (pending >> w) & 1u) {
          const uint4 a = ld_words(po + (size_t)w * L.slot_o + off);
          const uint4 b = ld_words(po + (size_t)w * L.slot_o + off + 16);
          const uint2 l2 = ld_word(pl + (size_t)w * L.slot_lse + (size_t)r * 8);
          if (a.y == step && a.w == step && b.y == step && b.w == step && l2.y == step) {
            pay[w][0] = a.x; pay[w][1] = a.z; pay[w][2] = b.x; pay[w][3] = b.z;
            lse_w[w] = __uint_as_float(l2.x);
            pending &= ~(1u << w);
          }
        }
      }
      if (pending && global_timer_ns() - t0 > kWaitLimitNs) { failed = true; break; }
    }
    if (failed) break;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kXMaxWorld; ++w)
      if (w < world) mx = fmaxf(mx, lse_w[w]);
    const float ms = mx == -INFINITY ? 0.f : mx;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float den = 0.f;
#pragma unroll
    for (int w = 0; w < kXMaxWorld; ++w) {
      if (w < world) {
        const float wt = __expf(lse_w[w] - ms);
        den += wt;
        if (wt != 0.f) {
          const T* e = reinterpret_cast<const T*>(&pay[w][0]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += wt * Elem<T>::to_f(e[j]);
        }
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    uint4 res;
    T* e = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = Elem<T>::from_f(acc[j] * inv);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(out) + (r * d + c * 8) * 2) = res;
    if (c == 0 && out_lse) out_lse[r] = den > 0.f ? ms + __logf(den) : -INFINITY;
  }
  if (__syncthreads_or(failed ? 1 : 0)) {
    if (tid == 0) record_wait_failure(wait_status, 601);
    return;
  }
  // ---- the last CTA to finish advances the step (every CTA has read it by then)
  if (tid == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(ctrl + 1, 1u) + 1u;
    if (done == gridDim.x) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctrl) = step;
    }
  }
}

}  // namespace

size_t xchg_buffer_bytes(int world, int64_t rows, int d) {
  if (world < 1 || world > kXMaxWorld || rows < 0 || d < 8 || d % 8) return 0;
  return xlayout(world, rows, d).total;
}

int xchg_grid(int64_t rows) {
  int64_t g = (rows + 15) / 16;       // >= 16 rows per CTA
  if (g > kXMaxGrid) g = kXMaxGrid;
  if (g < 1) g = 1;
  return (int)g;
}

int xchg_merge(const bsa_xchg_params* p, cudaStream_t s) {
  BSA_CHECK_ARG(p, "bsa_xchg_merge: null params");
  BSA_CHECK_ARG(p->world >= 1 && p->world <= kXMaxWorld && p->rank >= 0 && p->rank < p->world,
                "bsa_xchg_merge: bad world/rank %d/%d (at most %d ranks)", p->world, p->rank, kXMaxWorld);
  BSA_CHECK_ARG(p->rows >= 0 && p->d >= 8 && p->d % 8 == 0, "bsa_xchg_merge: bad sizes rows=%lld d=%d",
                (long long)p->rows, p->d);
  BSA_CHECK_ARG(p->dtype == BSA_F16 || p->dtype == BSA_BF16, "bsa_xchg_merge: partial outputs must be f16/bf16");
  BSA_CHECK_ARG(p->out && ((p->stage_o && p->stage_lse) || (p->part_o && p->part_lse && p->nsplit >= 1)),
                "bsa_xchg_merge: null pointer (merged rows, or split partials with nsplit >= 1)");
  XPtrs ptrs = {};
  for (int w = 0; w < p->world; ++w) {
    BSA_CHECK_ARG(p->xbuf[w] && reinterpret_cast<uintptr_t>(p->xbuf[w]) % 256 == 0,
                  "bsa_xchg_merge: exchange buffer %d is null or not 256-byte aligned", w);
    ptrs.buf[w] = static_cast<uint8_t*>(p->xbuf[w]);
  }
  BSA_CHECK_ARG(reinterpret_cast<uintptr_t>(p->stage_o) % 16 == 0 && reinterpret_cast<uintptr_t>(p->out) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(p->part_o) % 16 == 0,
                "bsa_xchg_merge: stage_o, part_o and out must be 16-byte aligned");
  if (p->rows == 0) return BSA_OK;
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  const int grid = xchg_grid(p->rows);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kXThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* part_o = p->stage_o ? nullptr : p->part_o;
  const float* part_lse = p->stage_o ? nullptr : p->part_lse;
  if (p->dtype == BSA_BF16)
    BSA_CHECK_CUDA(cudaLaunchKernelEx(&cfg, xchg_merge_kernel<__nv_bfloat16>, ptrs, (int)p->world, (int)p->rank,
                                      (int64_t)p->rows, (int)p->d, static_cast<const __nv_bfloat16*>(p->stage_o),
                                      p->stage_lse, part_o, part_lse, (int)p->nsplit,
                                      static_cast<__nv_bfloat16*>(p->out), p->out_lse, status));
  else
    BSA_CHECK_CUDA(cudaLaunchKernelEx(&cfg, xchg_merge_kernel<__half>, ptrs, (int)p->world, (int)p->rank,
                                      (int64_t)p->rows, (int)p->d, static_cast<const __half*>(p->stage_o),
                                      p->stage_lse, part_o, part_lse, (int)p->nsplit,
                                      static_cast<__half*>(p->out), p->out_lse, status));
  return check_launch("xchg_merge_kernel");
}

}  // namespace bsa
