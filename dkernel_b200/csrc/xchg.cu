// KV-sharded decode: exchange of the ranks' partial (O, LSE) rows and their merge, in ONE kernel
// per rank, over peer memory (NVLink) -- no library collective.
//
// Every rank owns an exchange buffer that all ranks of the node have mapped (CUDA IPC / symmetric
// memory; the host passes the W mapped addresses).  Per step, on every rank r:
//   phase 1  each CTA copies its rows of this rank's partial into slot r of EVERY rank's buffer
//            (ordinary 16-byte global stores, remote for the peers), fences at system scope and
//            stores the step number into its flag word in every rank's buffer (one writer per
//            flag, values only grow);
//   phase 2  the CTA waits until the W flag words of its own row range in the LOCAL buffer show
//            the current step, then merges the W partials of those rows with the semantics of
//            combine_attn_partitions (dkernel/interface.py:319-324) and writes the result.
// Only stores cross NVLink; every load is from local memory (L2-cached loads, because the lines
// are written by peers while the kernel runs).  A CTA depends on the same-numbered CTA of each
// peer only, and pushes before it waits, so the kernel cannot deadlock as long as CTAs are
// scheduled in index order; the wait is bounded (status word, as for the mbarrier waits).
// The step number lives in the buffer and is advanced by the last CTA to finish, so a captured
// CUDA graph can be replayed.  Slots are double buffered by step parity: a rank can be at most one
// step ahead of a peer (its next wait needs that peer's next push), so the slot it overwrites
// two steps later has been consumed.
#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kXThreads = 256;
constexpr int kXMaxGrid = 128;      // <= SM count: every CTA is resident
constexpr int kXMaxWorld = 8;

struct XLayout {
  size_t o_off, lse_off, flag_off, ctrl_off, total;
  size_t slot_o, slot_lse;   // bytes of one (parity, source rank) slot
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ inline XLayout xlayout(int world, int64_t rows, int d) {
  XLayout L;
  L.slot_o = align_up((size_t)rows * d * 2, 256);
  L.slot_lse = align_up((size_t)rows * 4, 256);
  L.o_off = 0;
  L.lse_off = L.o_off + 2 * (size_t)world * L.slot_o;
  L.flag_off = L.lse_off + 2 * (size_t)world * L.slot_lse;
  L.ctrl_off = L.flag_off + align_up((size_t)world * kXMaxGrid * 4, 256);
  L.total = L.ctrl_off + 256;
  return L;
}

struct XPtrs { uint8_t* buf[kXMaxWorld]; };

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kXThreads)
xchg_merge_kernel(XPtrs ptrs, int world, int rank, int64_t rows, int d, const T* __restrict__ stage_o,
                  const float* __restrict__ stage_lse, T* __restrict__ out, float* __restrict__ out_lse,
                  int* wait_status) {
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

  // ---- phase 1: this rank's rows -> slot `rank` of every rank's buffer
  for (int64_t i = tid; i < n_items; i += kXThreads) {
    const int64_t r = r0 + i / cpr;
    const int c = (int)(i % cpr);
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(stage_o) + (r * d + c * 8) * 2);
    const float l = c == 0 ? stage_lse[r] : 0.f;
    for (int w = 0; w < world; ++w) {
      uint8_t* dst = ptrs.buf[w];
      *reinterpret_cast<uint4*>(dst + L.o_off + (size_t)(par * world + rank) * L.slot_o + (r * d + c * 8) * 2) = v;
      if (c == 0)
        *reinterpret_cast<float*>(dst + L.lse_off + (size_t)(par * world + rank) * L.slot_lse + r * 4) = l;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world)
    st_release_sys(reinterpret_cast<uint32_t*>(ptrs.buf[tid] + L.flag_off) + rank * kXMaxGrid + cta, step);

  // ---- phase 2: wait for the same rows of every rank, then merge
  __shared__ int s_failed;
  if (tid == 0) s_failed = 0;
  __syncthreads();
  if (tid < world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + L.flag_off) + tid * kXMaxGrid + cta;
    const uint64_t t0 = global_timer_ns();
    bool ok = false;
    while (true) {
#pragma unroll 1
      for (int it = 0; it < 256 && !ok; ++it) ok = (int32_t)(ld_acquire_sys(flag) - step) >= 0;
      if (ok || global_timer_ns() - t0 > kWaitLimitNs) break;
    }
    if (!ok) s_failed = 1;
  }
  __syncthreads();
  if (s_failed) {
    if (tid == 0) record_wait_failure(wait_status, 601);
    return;
  }
  const uint8_t* po = mine + L.o_off + (size_t)par * world * L.slot_o;
  const uint8_t* pl = mine + L.lse_off + (size_t)par * world * L.slot_lse;
  for (int64_t i = tid; i < n_items; i += kXThreads) {
    const int64_t r = r0 + i / cpr;
    const int c = (int)(i % cpr);
    float lse_w[kXMaxWorld];
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kXMaxWorld; ++w) {
      if (w < world) {
        lse_w[w] = __ldcg(reinterpret_cast<const float*>(pl + (size_t)w * L.slot_lse) + r);
        mx = fmaxf(mx, lse_w[w]);
      }
    }
    const float ms = mx == -INFINITY ? 0.f : mx;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float den = 0.f;
#pragma unroll
    for (int w = 0; w < kXMaxWorld; ++w) {
      if (w < world) {
        const float wt = __expf(lse_w[w] - ms);
        den += wt;
        if (wt != 0.f) {
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(po + (size_t)w * L.slot_o + (r * d + c * 8) * 2));
          const T* e = reinterpret_cast<const T*>(&v);
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
  // ---- the last CTA to finish advances the step (every CTA has read it by then)
  __syncthreads();
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
  BSA_CHECK_ARG(p->stage_o && p->stage_lse && p->out, "bsa_xchg_merge: null pointer");
  XPtrs ptrs = {};
  for (int w = 0; w < p->world; ++w) {
    BSA_CHECK_ARG(p->xbuf[w] && reinterpret_cast<uintptr_t>(p->xbuf[w]) % 256 == 0,
                  "bsa_xchg_merge: exchange buffer %d is null or not 256-byte aligned", w);
    ptrs.buf[w] = static_cast<uint8_t*>(p->xbuf[w]);
  }
  BSA_CHECK_ARG(reinterpret_cast<uintptr_t>(p->stage_o) % 16 == 0 && reinterpret_cast<uintptr_t>(p->out) % 16 == 0,
                "bsa_xchg_merge: stage_o and out must be 16-byte aligned");
  if (p->rows == 0) return BSA_OK;
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  const int grid = xchg_grid(p->rows);
  if (p->dtype == BSA_BF16)
    xchg_merge_kernel<__nv_bfloat16><<<grid, kXThreads, 0, s>>>(
        ptrs, p->world, p->rank, p->rows, p->d, static_cast<const __nv_bfloat16*>(p->stage_o), p->stage_lse,
        static_cast<__nv_bfloat16*>(p->out), p->out_lse, status);
  else
    xchg_merge_kernel<__half><<<grid, kXThreads, 0, s>>>(
        ptrs, p->world, p->rank, p->rows, p->d, static_cast<const __half*>(p->stage_o), p->stage_lse,
        static_cast<__half*>(p->out), p->out_lse, status);
  return check_launch("xchg_merge_kernel");
}

}  // namespace bsa
