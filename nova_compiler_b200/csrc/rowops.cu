// HBM-bound companions of the contraction: layer_norm, softmax, gather, standalone activation and
// row-broadcast add.  Each reads its input from HBM once and writes its output once: a row lives
// in registers between the reduction and the normalisation pass (one warp per row up to 512 16-byte
// vectors = 4096 16-bit elements, with every load of the row issued before the first is consumed; one
// 256-thread CTA per row up to 4096 vectors; a two-pass loop beyond that), all traffic moves as 128-bit
// accesses when base and row pitch allow, and reductions are warp-shuffle trees.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "ptx_sm100.cuh"
#include "runtime.h"

namespace nova {
namespace {

template <typename T> __device__ __forceinline__ float ld_f32(T v);
template <> __device__ __forceinline__ float ld_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float ld_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T st_f32(float v);
template <> __device__ __forceinline__ float st_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half st_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 st_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T e[VEC]; };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduction over the TPR threads that share a row (TPR == 32: one warp; 64/128/256: that many
// consecutive threads of the CTA, i.e. TPR/32 consecutive warps, combined through shared memory).
template <int TPR, bool kMax>
__device__ __forceinline__ float row_reduce(float v, float* red_smem) {
  v = kMax ? warp_max(v) : warp_sum(v);
  if (TPR == 32) return v;
  constexpr int kWarpsPerRow = TPR / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = (warp / kWarpsPerRow) * kWarpsPerRow;  // first warp of this thread's row
  __syncthreads();  // protect red_smem from the previous reduction's readers
  if (lane == 0) red_smem[warp] = v;
  __syncthreads();
  float r = lane < kWarpsPerRow ? red_smem[first + lane] : (kMax ? -INFINITY : 0.0f);
  return kMax ? warp_max(r) : warp_sum(r);
}

// Two values at once, ONE barrier per call: the exchange buffer alternates between calls (`phase`), so a warp
// writes buffer b only after every thread has passed the barrier of the call before, i.e. after all readers of
// the call before that (the last user of b) are done.  Lowers the barriers of a layer_norm row from four to one.
template <int TPR, bool kMax>
__device__ __forceinline__ void row_reduce2(float& a, float& b, float2 (*red_smem)[8], uint32_t& phase) {
  a = kMax ? warp_max(a) : warp_sum(a);
  b = kMax ? warp_max(b) : warp_sum(b);
  if (TPR == 32) return;
  constexpr int kWarpsPerRow = TPR / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = (warp / kWarpsPerRow) * kWarpsPerRow;
  float2* buf = red_smem[phase & 1u];
  ++phase;
  if (lane == 0) buf[warp] = make_float2(a, b);
  __syncthreads();
  const float2 r = lane < kWarpsPerRow ? buf[first + lane] : (kMax ? make_float2(-INFINITY, -INFINITY) : make_float2(0.0f, 0.0f));
  a = kMax ? warp_max(r.x) : warp_sum(r.x);
  b = kMax ? warp_max(r.y) : warp_sum(r.y);
}

constexpr int kRowThreads = 256;
constexpr int kLongUnroll = 8;
inline bool ring_rows_enabled() { return options().ring_rows.load() != 0; }  // vectors a thread keeps in flight when a row is too long for its registers

// kMode 0: layer_norm, kMode 1: softmax.  kMaxV > 0: a thread keeps up to kMaxV vectors of its row in
// registers (the row fits TPR * kMaxV vectors); kMaxV == 0: two passes over global memory.  kMaxV is
// picked as small as the row allows so that short rows leave registers for more resident warps.
template <typename T, int VEC, int TPR, int kMaxV, int kMode>
__global__ void __launch_bounds__(kRowThreads, (VEC > 1 && kMaxV > 0 && kMaxV <= 2) ? 6 : (VEC > 1 && kMaxV == 4 ? 5 : 1))
row_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
           T* __restrict__ mean_sum, T* __restrict__ rstd_out, int64_t rows, int32_t D, int32_t prefetch_next,
           float* __restrict__ row_stats) {  // softmax only, optional: {row max, sum of exp(x - max)} per row
  __shared__ float2 red2[2][8];
  static_assert(kRowThreads / 32 == 8, "exchange buffer size");
  uint32_t red_phase = 0;
  constexpr int kRowsPerCta = kRowThreads / TPR;
  constexpr bool CACHED = kMaxV > 0;
  const int t = threadIdx.x % TPR;
  const int sub = threadIdx.x / TPR;
  const int nvec = D / VEC;  // host guarantees D % VEC == 0
  using P = Pack<T, VEC>;
  const float inv_d = 1.0f / static_cast<float>(D);

  // Persistent CTAs walk the rows.  Before a row is reduced, the CTA's NEXT row is prefetched into L2
  // (one request per 128-byte line, no registers held), so HBM reads stay in flight through the
  // reduction and store phases and the next row's loads are L2 hits.
  const int64_t row_step = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta; row0 < rows; row0 += row_step) {
    const int64_t row = row0 + sub;
    const bool active = row < rows;  // uniform over the TPR threads of a row
    const P* xr = reinterpret_cast<const P*>(x + (active ? row : 0) * D);
    P* yr = reinterpret_cast<P*>(y + (active ? row : 0) * D);
    P cache[CACHED ? kMaxV : 1];  // all the row's loads are issued before the first is consumed
    if (prefetch_next && row + row_step < rows) {
      const P* nx = reinterpret_cast<const P*>(x + (row + row_step) * D);
      constexpr int kVecPerLine = 128 / static_cast<int>(sizeof(P));
      for (int i = t * kVecPerLine; i < nvec; i += TPR * kVecPerLine)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + i));
    }

    float s0 = kMode == 0 ? 0.0f : -INFINITY;  // layer_norm: sum; softmax: max
    float s1 = 0.0f;                            // layer_norm: sum of squares; long softmax rows: running sum of exp
    if (CACHED) {
#pragma unroll
      for (int k = 0; k < kMaxV; ++k) {
        const int i = t + k * TPR;
        if (active && i < nvec) {
          cache[k] = xr[i];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float v = ld_f32<T>(cache[k].e[e]);
            if (kMode == 0) { s0 += v; s1 += v * v; } else { s0 = fmaxf(s0, v); }
          }
        }
      }
    } else {
      // kLongUnroll independent loads per thread and trip: long rows run on few CTAs, so the bytes in flight
      // have to come from each thread
      for (int i0 = t; active && i0 < nvec; i0 += TPR * kLongUnroll) {
        P pks[kLongUnroll];
#pragma unroll
        for (int u = 0; u < kLongUnroll; ++u)
          if (i0 + u * TPR < nvec) pks[u] = xr[i0 + u * TPR];
#pragma unroll
        for (int u = 0; u < kLongUnroll; ++u) {
        if (i0 + u * TPR >= nvec) break;
        const P pk = pks[u];
        if (kMode == 0) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float v = ld_f32<T>(pk.e[e]);
            s0 += v;
            s1 += v * v;
          }
        } else {
          // online softmax: the running sum is kept relative to the running maximum, so the row is read once here
          float vm = ld_f32<T>(pk.e[0]);
#pragma unroll
          for (int e = 1; e < VEC; ++e) vm = fmaxf(vm, ld_f32<T>(pk.e[e]));
          if (vm > s0) { s1 *= __expf(s0 - vm); s0 = vm; }
#pragma unroll
          for (int e = 0; e < VEC; ++e) s1 += __expf(ld_f32<T>(pk.e[e]) - s0);
        }
        }
      }
    }

    if (kMode == 0) {
      row_reduce2<TPR, false>(s0, s1, red2, red_phase);
      const float sum = s0, sq = s1;
      const float mean = sum * inv_d;
      const float var = sq * inv_d - mean * mean;
      const float rstd = rsqrtf(var + 1e-5f);
      if (active && t == 0) {
        if (mean_sum) mean_sum[row] = st_f32<T>(sum);
        if (rstd_out) rstd_out[row] = st_f32<T>(rstd);
      }
      const P* gr = reinterpret_cast<const P*>(gamma);
      const P* br = reinterpret_cast<const P*>(beta);
      auto emit = [&](int i, const P& in) {
        const P g = gr[i], b = br[i];
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          o.e[e] = st_f32<T>((ld_f32<T>(in.e[e]) - mean) * rstd * ld_f32<T>(g.e[e]) + ld_f32<T>(b.e[e]));
        yr[i] = o;
      };
      if (CACHED) {
#pragma unroll
        for (int k = 0; k < kMaxV; ++k) {
          const int i = t + k * TPR;
          if (active && i < nvec) emit(i, cache[k]);
        }
      } else {
        for (int i0 = t; active && i0 < nvec; i0 += TPR * kLongUnroll) {
          P pks[kLongUnroll];
#pragma unroll
          for (int u = 0; u < kLongUnroll; ++u)
            if (i0 + u * TPR < nvec) pks[u] = xr[i0 + u * TPR];
#pragma unroll
          for (int u = 0; u < kLongUnroll; ++u)
            if (i0 + u * TPR < nvec) emit(i0 + u * TPR, pks[u]);
        }
      }
    } else {
      float m = s0, m_dup = 0.0f;
      if (TPR == 32) m = warp_max(m);
      else row_reduce2<TPR, true>(m, m_dup, red2, red_phase);
      float part = 0.0f;
      if (!CACHED) part = s0 == -INFINITY ? 0.0f : s1 * __expf(s0 - m);  // this thread's sum, rescaled to the row max
      if (CACHED) {
#pragma unroll
        for (int k = 0; k < kMaxV; ++k) {
          const int i = t + k * TPR;
          if (active && i < nvec) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) part += __expf(ld_f32<T>(cache[k].e[e]) - m);
          }
        }
      }
      float s = part, s_dup = 0.0f;
      if (TPR == 32) s = warp_sum(s);
      else row_reduce2<TPR, false>(s, s_dup, red2, red_phase);
      if (row_stats != nullptr && active && t == 0) { row_stats[2 * row] = m; row_stats[2 * row + 1] = s; }
      const float recip = 1.0f / fmaxf(s, 1.0e-7f);
      auto emit = [&](int i, const P& in) {
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.e[e] = st_f32<T>(__expf(ld_f32<T>(in.e[e]) - m) * recip);
        yr[i] = o;
      };
      if (CACHED) {
#pragma unroll
        for (int k = 0; k < kMaxV; ++k) {
          const int i = t + k * TPR;
          if (active && i < nvec) emit(i, cache[k]);
        }
      } else {
        for (int i0 = t; active && i0 < nvec; i0 += TPR * kLongUnroll) {
          P pks[kLongUnroll];
#pragma unroll
          for (int u = 0; u < kLongUnroll; ++u)
            if (i0 + u * TPR < nvec) pks[u] = xr[i0 + u * TPR];
#pragma unroll
          for (int u = 0; u < kLongUnroll; ++u)
            if (i0 + u * TPR < nvec) emit(i0 + u * TPR, pks[u]);
        }
      }
    }
  }
}

// cudaFuncSetAttribute + the occupancy query cost microseconds each: the attribute is raised once per kernel instance
// (to the most any ring may ask for), the occupancy is looked up once per ring size, per host thread.
constexpr size_t kRingMaxBytes = 200u << 10;

// (keyed on the kernel's address: instances that differ only in a template argument share one function-pointer type)
template <typename Kernel>
int ring_resident_ctas(Kernel kernel, int threads, size_t smem) {
  struct Entry { const void* fn; int device; size_t smem; int resident; };
  static thread_local Entry cache[32] = {};
  static thread_local int used = 0;
  const void* fn = reinterpret_cast<const void*>(kernel);
  if (smem > kRingMaxBytes) { set_error("ring of " + std::to_string(smem) + " bytes exceeds the limit"); return 0; }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); set_error("cudaGetDevice failed"); return 0; }
  bool configured = false;  // (a function attribute belongs to one device's copy of the kernel)
  for (int i = 0; i < used; ++i) {
    if (cache[i].fn != fn || cache[i].device != device) continue;
    configured = true;
    if (cache[i].smem == smem) return cache[i].resident;
  }
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRingMaxBytes));
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
      return 0;
    }
  }
  int resident = 0;
  const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, threads, smem);
  if (e != cudaSuccess || resident <= 0) {
    cudaGetLastError();
    set_error(std::string("occupancy query: ") + cudaGetErrorString(e) + ", resident " + std::to_string(resident) + ", smem " + std::to_string(smem));
    return 0;
  }
  cache[used < 32 ? used++ : 31] = Entry{fn, device, smem, resident};
  return resident;
}

// ---------------------------------------------------------------- layer_norm rows through a shared-memory ring
//
// For rows of a few KB (one 256-thread CTA per row) the register-cached kernels above are latency-bound: a CTA's
// loads, reduction and stores of one row are serial, and the bytes in flight per SM are what its resident CTAs
// hold in registers.  Here the rows of a persistent CTA stream through a ring of kStages shared-memory slots
// filled by bulk copies (cp.async.bulk, completion counted on an mbarrier): kStages - 1 rows per CTA are in flight
// while one is being reduced, no registers are held for them, and a row costs ONE CTA barrier (the pair reduction,
// after which the slot is free and thread 0 refills it at once).  y is written straight from registers.
//
// Waits are bounded: a thread that gives up records kStatusRowRingWait, raises the CTA's abort flag BEFORE the
// row's barrier and every thread leaves after it, so the decision is uniform; in-flight copies are then given time to land.
constexpr uint32_t kStatusRowRingWait = 0x201;
constexpr uint32_t kRingSpinLimit = 1u << 24;

// ---- two elements per instruction: sm_100's packed fp32 pipe (fma/add/mul on float2) halves the issue slots of the
// arithmetic, which is what bounds these kernels (their DRAM traffic is already the algorithmic minimum).
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
// Pair `P` of a 16-byte vector of T as two floats (16-bit types: one 32-bit word; float: two words).
template <typename T, int P> __device__ __forceinline__ float2 pair_of(const uint4& v);
#define NOVA_WORD(v, i) ((i) == 0 ? (v).x : (i) == 1 ? (v).y : (i) == 2 ? (v).z : (v).w)
template <typename T, int P> __device__ __forceinline__ float2 pair_of(const uint4& v) {
  if constexpr (sizeof(T) == 4) {
    return make_float2(__uint_as_float(NOVA_WORD(v, 2 * P)), __uint_as_float(NOVA_WORD(v, 2 * P + 1)));
  } else if constexpr (std::is_same<T, __half>::value) {
    const uint32_t w = NOVA_WORD(v, P);
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  } else {
    const uint32_t w = NOVA_WORD(v, P);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
}
#undef NOVA_WORD
// Two floats rounded to T, as the 32-bit word (16-bit types) they occupy in a vector.
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float2 v) {
  if constexpr (std::is_same<T, __half>::value) {
    const __half2 h = __float22half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    const __nv_bfloat162 h = __float22bfloat162_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}

// Sums N (a power of two, <= 32) values over the warp in N - 1 + log2(32 / N) shuffles instead of 5 N: each
// exchange step halves the values a lane still carries (the lane keeps one half of the set and hands the other to its
// partner).  Returns the complete sum number `j` (also returned), the same in the 32 / N lanes that share it.
template <int N>
__device__ __forceinline__ float warp_multi_sum(float (&v)[N], int lane, int& j) {
  int off = 16;
  j = 0;
#pragma unroll
  for (int n = N; n > 1; n >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = up ? v[i] : v[i + n / 2];
      const float keep = up ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    j += up ? n / 2 : 0;
    off >>= 1;
  }
#pragma unroll
  for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
  return v[0];
}

// f(p, pair p of `v` as two floats) for every element pair of a 16-byte vector of T.
template <typename T, typename F>
__device__ __forceinline__ void for_pairs(const uint4& v, F&& f) {
  f(0, pair_of<T, 0>(v));
  f(1, pair_of<T, 1>(v));
  if constexpr (sizeof(T) == 2) {
    f(2, pair_of<T, 2>(v));
    f(3, pair_of<T, 3>(v));
  }
}
// Pair `p` of the 16-byte vector assembled in `w`, rounded to T.
template <typename T>
__device__ __forceinline__ void put_pair(uint32_t (&w)[4], int p, float2 v) {
  if constexpr (sizeof(T) == 4) {
    w[2 * p] = __float_as_uint(v.x);
    w[2 * p + 1] = __float_as_uint(v.y);
  } else {
    w[p] = pack_pair<T>(v);
  }
}

// Two sums over the 256 threads of a CTA with one barrier (exchange buffer alternating per call, as row_reduce2):
// the warp stage halves the carried values after the first exchange (6 shuffles instead of 10).
__device__ __forceinline__ void cta256_sum2(float& a, float& b, float2 (*red_smem)[8], uint32_t& phase) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float v[2] = {a, b};
  int j;
  const float m = warp_multi_sum<2>(v, lane, j);
  float* buf = reinterpret_cast<float*>(red_smem[phase & 1u]);
  ++phase;
  if ((lane & 15) == 0) buf[2 * warp + j] = m;
  __syncthreads();
  float2 r = reinterpret_cast<const float2*>(buf)[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    r.x += __shfl_xor_sync(0xffffffffu, r.x, o);
    r.y += __shfl_xor_sync(0xffffffffu, r.y, o);
  }
  a = r.x;
  b = r.y;
}

// softmax of rows that fit one warp's registers (at most 32 * kMaxV 16-byte vectors), one warp per row, no CTA barrier.
// exp(x - max) is evaluated ONCE per element and kept in fp32 registers for the normalisation (the special-function
// unit retires 16 results per SM and cycle: two evaluations per element would cost more than the row's HBM time), the
// row maximum is taken on the packed 16-bit words, and the remaining arithmetic is packed fp32.  Lanes past the row
// carry -inf (exp gives 0) so that no arithmetic is predicated.
template <typename T, int kMaxV>
__global__ void __launch_bounds__(kRowThreads)
softmax_warp_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t D, float* __restrict__ row_stats) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T)), NP = VEC / 2, kRowsPerCta = kRowThreads / 32;
  const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
  const int nvec = D / VEC;
  const uint32_t ninf = sizeof(T) == 4 ? 0xff800000u : std::is_same<T, __half>::value ? 0xfc00fc00u : 0xff80ff80u;
  const uint4 fill = make_uint4(ninf, ninf, ninf, ninf);
  const int64_t step = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + sub; row < rows; row += step) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
    uint4 cache[kMaxV];
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) cache[k] = lane + 32 * k < nvec ? xr[lane + 32 * k] : fill;
    float m;
    if constexpr (sizeof(T) == 4) {
      m = -INFINITY;
#pragma unroll
      for (int k = 0; k < kMaxV; ++k)
        m = fmaxf(fmaxf(m, fmaxf(__uint_as_float(cache[k].x), __uint_as_float(cache[k].y))),
                  fmaxf(__uint_as_float(cache[k].z), __uint_as_float(cache[k].w)));
    } else {
      using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
      auto as2 = [](uint32_t w) { return *reinterpret_cast<const T2*>(&w); };
      T2 mm = as2(ninf);
#pragma unroll
      for (int k = 0; k < kMaxV; ++k)
        mm = __hmax2(__hmax2(mm, __hmax2(as2(cache[k].x), as2(cache[k].y))), __hmax2(as2(cache[k].z), as2(cache[k].w)));
      const uint32_t w = *reinterpret_cast<const uint32_t*>(&mm);
      const float2 f = pair_of<T, 0>(make_uint4(w, 0u, 0u, 0u));
      m = fmaxf(f.x, f.y);
    }
    m = warp_max(m);
    const float2 neg_m = splat2(-m), log2e = splat2(1.4426950408889634f);
    float2 e[kMaxV][NP];
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      for_pairs<T>(cache[k], [&](int p, float2 v) {
        const float2 a = __fmul2_rn(__fadd2_rn(v, neg_m), log2e);
        float2 r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(a.x));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(a.y));
        e[k][p] = r;
        acc = __fadd2_rn(acc, r);
      });
    }
    const float total = warp_sum(acc.x + acc.y);
    if (row_stats != nullptr && lane == 0) { row_stats[2 * row] = m; row_stats[2 * row + 1] = total; }
    const float2 recip = splat2(1.0f / fmaxf(total, 1.0e-7f));
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      uint32_t w[4];
#pragma unroll
      for (int p = 0; p < NP; ++p) put_pair<T>(w, p, __fmul2_rn(e[k][p], recip));
      if (lane + 32 * k < nvec) yr[lane + 32 * k] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// layer_norm of rows that fit one warp's registers (at most 32 * kMaxV 16-byte vectors; 2 KB for kMaxV = 4), one warp
// per row, no CTA barrier, packed fp32 arithmetic; the row's two sums cross the warp in one six-shuffle tree.  gamma
// and beta are re-read per row (L1 hits): a warp's registers hold the row, not the parameters.
template <typename T, int kMaxV>
__global__ void __launch_bounds__(kRowThreads)
ln_warp_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
               T* __restrict__ mean_sum, T* __restrict__ rstd_out, int64_t rows, int32_t D) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T)), kRowsPerCta = kRowThreads / 32;
  const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
  const int nvec = D / VEC;
  const float inv_d = 1.0f / static_cast<float>(D);
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
  const uint4* b4 = reinterpret_cast<const uint4*>(beta);
  const int64_t step = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + sub; row < rows; row += step) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
    uint4 cache[kMaxV];
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) cache[k] = lane + 32 * k < nvec ? xr[lane + 32 * k] : zero4;  // zeros add nothing
    float2 a0 = make_float2(0.0f, 0.0f), a1 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k)
      for_pairs<T>(cache[k], [&](int, float2 v) {
        a0 = __fadd2_rn(a0, v);
        a1 = __ffma2_rn(v, v, a1);
      });
    float v2[2] = {a0.x + a0.y, a1.x + a1.y};
    int j;
    const float mine = warp_multi_sum<2>(v2, lane, j);   // lanes 0-15 hold the sum, lanes 16-31 the sum of squares
    const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
    const float s0 = j == 0 ? mine : other, s1 = j == 0 ? other : mine;
    const float mean = s0 * inv_d;
    const float rstd = rsqrtf(s1 * inv_d - mean * mean + 1e-5f);
    if (lane == 0) {
      if (mean_sum) mean_sum[row] = st_f32<T>(s0);
      if (rstd_out) rstd_out[row] = st_f32<T>(rstd);
    }
    const float2 rs2 = splat2(rstd), nm2 = splat2(-mean * rstd);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = lane + 32 * k;
      if (i < nvec) {
        const uint4 gr = g4[i], br = b4[i];
        float2 gk[VEC / 2], bk[VEC / 2];
        for_pairs<T>(gr, [&](int p, float2 v) { gk[p] = v; });
        for_pairs<T>(br, [&](int p, float2 v) { bk[p] = v; });
        uint32_t w[4];
        for_pairs<T>(cache[k], [&](int p, float2 v) { put_pair<T>(w, p, __ffma2_rn(__ffma2_rn(v, rs2, nm2), gk[p], bk[p])); });
        yr[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

// One lane per warp polls (these kernels are bound by instruction issue, and 32 lanes spinning on one barrier are
// 32 times the instructions); the warp reconverges on __syncwarp, which also orders the lanes' later reads of the slot
// after the observed completion.
__device__ __forceinline__ void ring_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
  if ((threadIdx.x & 31) == 0) {
    bool done = false;
    for (uint32_t it = 0; it < kRingSpinLimit && !done; ++it) done = mbar_try_wait(bar, parity);
    if (!done) {
      *abort_flag = 1u;
      atomicCAS(status, 0u, kStatusRowRingWait);
    }
  }
  __syncwarp();
}

constexpr int kRingMaxStages = 8;

template <typename T, int kMaxV>
__global__ void __launch_bounds__(kRowThreads)
ln_ring_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
               T* __restrict__ mean_sum, T* __restrict__ rstd_out, int64_t rows, int32_t D, int32_t kStages,
               uint32_t* status) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[kRingMaxStages];
  __shared__ __align__(16) float2 red2[2][8];
  __shared__ uint32_t abort_smem;
  volatile uint32_t* abort_flag = &abort_smem;
  uint32_t red_phase = 0;
  const int t = threadIdx.x;
  const int nvec = D / VEC;
  const uint32_t row_bytes = static_cast<uint32_t>(D) * sizeof(T);
  const float inv_d = 1.0f / static_cast<float>(D);
  if (t == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&full[s]), 1);
    abort_smem = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  const int64_t step = gridDim.x;
  if (t == 0) {
    for (int s = 0; s < kStages; ++s) {
      const int64_t r = blockIdx.x + s * step;
      if (r < rows) {
        mbar_arrive_expect_tx(smem_u32(&full[s]), row_bytes);
        bulk_load(smem_u32(ring + static_cast<size_t>(s) * row_bytes), x + r * D, row_bytes, smem_u32(&full[s]));
      }
    }
  }
  // short rows keep their gamma / beta vectors in registers (as floats: no conversion per row); longer ones re-read
  // them (L1 / L2 hits) to stay at a register count that lets several CTAs share an SM.  Arithmetic is packed fp32.
  constexpr bool kPreload = kMaxV <= 2;
  constexpr int NP = VEC / 2;
  float2 gf[kPreload ? kMaxV : 1][NP], bf[kPreload ? kMaxV : 1][NP];
  if (kPreload) {
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kRowThreads;
      const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
      const uint4 gr = i < nvec ? reinterpret_cast<const uint4*>(gamma)[i] : zero4;
      const uint4 br = i < nvec ? reinterpret_cast<const uint4*>(beta)[i] : zero4;
      for_pairs<T>(gr, [&](int p, float2 v) { gf[kPreload ? k : 0][p] = v; });
      for_pairs<T>(br, [&](int p, float2 v) { bf[kPreload ? k : 0][p] = v; });
    }
  }
  uint32_t it = 0;
  for (int64_t row = blockIdx.x; row < rows; row += step, ++it) {
    const int s = it % kStages;
    ring_wait(smem_u32(&full[s]), (it / kStages) & 1u, abort_flag, status);
    const uint4* slot = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(s) * row_bytes);
    uint4 cache[kMaxV];
    float2 a0 = make_float2(0.0f, 0.0f), a1 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kRowThreads;
      if (i < nvec) {
        cache[k] = slot[i];
        for_pairs<T>(cache[k], [&](int, float2 v) {
          a0 = __fadd2_rn(a0, v);
          a1 = __ffma2_rn(v, v, a1);
        });
      }
    }
    float s0 = a0.x + a0.y, s1 = a1.x + a1.y;
    cta256_sum2(s0, s1, red2, red_phase);   // one barrier: every thread has read the slot
    if (*abort_flag != 0u) break;           // (raised before the barrier: all threads see it)
    if (t == 0) {
      const int64_t nr = row + kStages * step;
      if (nr < rows) {
        mbar_arrive_expect_tx(smem_u32(&full[s]), row_bytes);
        bulk_load(smem_u32(ring + static_cast<size_t>(s) * row_bytes), x + nr * D, row_bytes, smem_u32(&full[s]));
      }
    }
    const float mean = s0 * inv_d;
    const float rstd = rsqrtf(s1 * inv_d - mean * mean + 1e-5f);
    if (t == 0) {
      if (mean_sum) mean_sum[row] = st_f32<T>(s0);
      if (rstd_out) rstd_out[row] = st_f32<T>(rstd);
    }
    const float2 rs2 = splat2(rstd), nm2 = splat2(-mean * rstd);
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kRowThreads;
      if (i < nvec) {
        uint32_t w[4];
        if (kPreload) {
          for_pairs<T>(cache[k], [&](int p, float2 v) {
            put_pair<T>(w, p, __ffma2_rn(__ffma2_rn(v, rs2, nm2), gf[kPreload ? k : 0][p], bf[kPreload ? k : 0][p]));
          });
        } else {
          const uint4 gr = reinterpret_cast<const uint4*>(gamma)[i], br = reinterpret_cast<const uint4*>(beta)[i];
          float2 gk[NP], bk[NP];
          for_pairs<T>(gr, [&](int p, float2 v) { gk[p] = v; });
          for_pairs<T>(br, [&](int p, float2 v) { bk[p] = v; });
          for_pairs<T>(cache[k], [&](int p, float2 v) {
            put_pair<T>(w, p, __ffma2_rn(__ffma2_rn(v, rs2, nm2), gk[p], bk[p]));
          });
        }
        yr[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  if (*abort_flag != 0u && t == 0)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let copies still in flight land before the CTA's memory is reused
  __syncthreads();
}

// One value over the 256 threads of a CTA, one barrier (exchange buffer alternating per call).
template <bool kMax>
__device__ __forceinline__ float cta256_reduce1(float v, float (*buf)[8], uint32_t& phase) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  v = kMax ? warp_max(v) : warp_sum(v);
  float* b = buf[phase & 1u];
  ++phase;
  if (lane == 0) b[warp] = v;
  __syncthreads();
  float r = b[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    const float q = __shfl_xor_sync(0xffffffffu, r, o);
    r = kMax ? fmaxf(r, q) : r + q;
  }
  return r;
}

// softmax rows of 4-32 KB through the same ring as ln_ring_kernel: a persistent 256-thread CTA, row slots filled by
// bulk copies, the row's vectors in registers after the first read.  Two CTA barriers per row (maximum, sum); the slot
// is refilled after the first.  exp is evaluated once per element where the values fit in registers as floats (fp32
// rows; 16-bit rows of up to 512 vectors), else once for the sum and once for the output; packed fp32 arithmetic.
template <typename T, int kMaxV>
__global__ void __launch_bounds__(kRowThreads)
softmax_ring_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t D, int32_t kStages,
                    float* __restrict__ row_stats, uint32_t* status) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T)), NP = VEC / 2;
  constexpr bool kKeep = sizeof(T) == 4 || kMaxV <= 2;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[kRingMaxStages];
  __shared__ float red[2][8];
  __shared__ uint32_t abort_smem;
  volatile uint32_t* abort_flag = &abort_smem;
  uint32_t red_phase = 0;
  const int t = threadIdx.x;
  const int nvec = D / VEC;
  const uint32_t row_bytes = static_cast<uint32_t>(D) * sizeof(T);
  if (t == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&full[s]), 1);
    abort_smem = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  const int64_t step = gridDim.x;
  if (t == 0) {
    for (int s = 0; s < kStages; ++s) {
      const int64_t r = blockIdx.x + s * step;
      if (r < rows) {
        mbar_arrive_expect_tx(smem_u32(&full[s]), row_bytes);
        bulk_load(smem_u32(ring + static_cast<size_t>(s) * row_bytes), x + r * D, row_bytes, smem_u32(&full[s]));
      }
    }
  }
  const uint32_t ninf = sizeof(T) == 4 ? 0xff800000u : std::is_same<T, __half>::value ? 0xfc00fc00u : 0xff80ff80u;
  const uint4 fill = make_uint4(ninf, ninf, ninf, ninf);  // vectors past the row: exp gives 0
  const float2 log2e = splat2(1.4426950408889634f);
  uint32_t it = 0;
  for (int64_t row = blockIdx.x; row < rows; row += step, ++it) {
    const int s = it % kStages;
    ring_wait(smem_u32(&full[s]), (it / kStages) & 1u, abort_flag, status);
    const uint4* slot = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(s) * row_bytes);
    uint4 cache[kMaxV];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kRowThreads;
      cache[k] = i < nvec ? slot[i] : fill;
      for_pairs<T>(cache[k], [&](int, float2 f) { m = fmaxf(m, fmaxf(f.x, f.y)); });
    }
    m = cta256_reduce1<true>(m, red, red_phase);   // every thread has read the slot
    if (*abort_flag != 0u) break;                  // (raised before the barrier: all threads see it)
    if (t == 0) {
      const int64_t nr = row + kStages * step;
      if (nr < rows) {
        mbar_arrive_expect_tx(smem_u32(&full[s]), row_bytes);
        bulk_load(smem_u32(ring + static_cast<size_t>(s) * row_bytes), x + nr * D, row_bytes, smem_u32(&full[s]));
      }
    }
    const float2 neg_m = splat2(-m);
    auto exp_of = [&](float2 f) {
      const float2 a = __fmul2_rn(__fadd2_rn(f, neg_m), log2e);
      float2 e;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(a.x));
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(a.y));
      return e;
    };
    float2 e[kKeep ? kMaxV : 1][NP];
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k)
      for_pairs<T>(cache[k], [&](int p, float2 f) {
        const float2 v = exp_of(f);
        acc = __fadd2_rn(acc, v);
        if (kKeep) e[kKeep ? k : 0][p] = v;
      });
    const float total = cta256_reduce1<false>(acc.x + acc.y, red, red_phase);
    if (row_stats != nullptr && t == 0) { row_stats[2 * row] = m; row_stats[2 * row + 1] = total; }
    const float2 recip = splat2(1.0f / fmaxf(total, 1.0e-7f));
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kRowThreads;
      uint32_t w[4];
      if (kKeep) {
#pragma unroll
        for (int p = 0; p < NP; ++p) put_pair<T>(w, p, __fmul2_rn(e[kKeep ? k : 0][p], recip));
      } else {
        for_pairs<T>(cache[k], [&](int p, float2 f) { put_pair<T>(w, p, __fmul2_rn(exp_of(f), recip)); });
      }
      if (i < nvec) yr[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (*abort_flag != 0u && t == 0)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let copies still in flight land before the CTA's memory is reused
  __syncthreads();
}

// layer_norm_backward the same way: a slot holds one row of grad_y and one of x (two bulk copies, one barrier
// phase); a thread owns the same vectors of every row, so dgamma / dbeta accumulate in its registers and leave as
// one partial row per CTA; the next row's mean and rstd are fetched a row ahead.
template <typename T, int kMaxV, int kThreads>
__global__ void __launch_bounds__(kThreads, kMaxV == 1 ? 2 : 1)
ln_backward_ring_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ gamma,
                        const T* __restrict__ mean_sum, const T* __restrict__ rstd, T* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows, int32_t D, int32_t kStages, uint32_t* status) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  using P = Pack<T, VEC>;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[kRingMaxStages];
  __shared__ float2 red2[2][kThreads / 32];
  __shared__ uint32_t abort_smem;
  volatile uint32_t* abort_flag = &abort_smem;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  constexpr int kWarps = kThreads / 32;
  const int nvec = D / VEC;
  const uint32_t row_bytes = static_cast<uint32_t>(D) * sizeof(T);
  const float inv_d = 1.0f / static_cast<float>(D);
  if (t == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&full[s]), 1);
    abort_smem = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  const int64_t step = gridDim.x;
  auto fill = [&](int s, int64_t r) {
    const uint32_t bar = smem_u32(&full[s]);
    uint8_t* dst = ring + static_cast<size_t>(s) * 2 * row_bytes;
    mbar_arrive_expect_tx(bar, 2 * row_bytes);
    bulk_load(smem_u32(dst), gy + r * D, row_bytes, bar);
    bulk_load(smem_u32(dst + row_bytes), x + r * D, row_bytes, bar);
  };
  if (t == 0)
    for (int s = 0; s < kStages; ++s)
      if (blockIdx.x + s * step < rows) fill(s, blockIdx.x + s * step);
  P gam[kMaxV];
  float dg[kMaxV][VEC], db[kMaxV][VEC];
#pragma unroll
  for (int k = 0; k < kMaxV; ++k) {
    const int i = t + k * kThreads;
    if (i < nvec) gam[k] = reinterpret_cast<const P*>(gamma)[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) dg[k][e] = db[k][e] = 0.0f;
  }
  float mean_next = 0.0f, rs_next = 0.0f;
  if (static_cast<int64_t>(blockIdx.x) < rows) {
    mean_next = ld_f32<T>(mean_sum[blockIdx.x]) * inv_d;
    rs_next = ld_f32<T>(rstd[blockIdx.x]);
  }
  uint32_t it = 0;
  for (int64_t row = blockIdx.x; row < rows; row += step, ++it) {
    const int s = it % kStages;
    const float mean = mean_next, rs = rs_next;
    if (row + step < rows) {
      mean_next = ld_f32<T>(mean_sum[row + step]) * inv_d;
      rs_next = ld_f32<T>(rstd[row + step]);
    }
    ring_wait(smem_u32(&full[s]), (it / kStages) & 1u, abort_flag, status);
    const P* sg = reinterpret_cast<const P*>(ring + static_cast<size_t>(s) * 2 * row_bytes);
    const P* sx = reinterpret_cast<const P*>(ring + static_cast<size_t>(s) * 2 * row_bytes + row_bytes);
    // xhat and gy * gamma stay in registers as floats across the row's barrier: the second half of the row is then
    // three operations per element instead of a second round of conversions
    float xh[kMaxV][VEC], gg[kMaxV][VEC];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kThreads;
      if (i < nvec) {
        const P pg = sg[i], px = sx[i];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float g = ld_f32<T>(pg.e[e]);
          const float xhat = (ld_f32<T>(px.e[e]) - mean) * rs;
          const float gyg = g * ld_f32<T>(gam[k].e[e]);
          xh[k][e] = xhat;
          gg[k][e] = gyg;
          s1 += gyg;
          s2 = fmaf(gyg, xhat, s2);
          dg[k][e] = fmaf(g, xhat, dg[k][e]);
          db[k][e] += g;
        }
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    float2* buf = red2[it & 1u];  // alternating exchange buffer: one barrier per row
    if (lane == 0) buf[warp] = make_float2(s1, s2);
    __syncthreads();
    if (*abort_flag != 0u) break;
    if (t == 0 && row + kStages * step < rows) fill(s, row + kStages * step);  // every thread has read the slot
    const float2 r2 = lane < kWarps ? buf[lane] : make_float2(0.0f, 0.0f);
    const float m1 = warp_sum(r2.x) * inv_d, m2 = warp_sum(r2.y) * inv_d;
    P* dxr = reinterpret_cast<P*>(dx + row * D);
#pragma unroll
    for (int k = 0; k < kMaxV; ++k) {
      const int i = t + k * kThreads;
      if (i < nvec) {
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.e[e] = st_f32<T>(((gg[k][e] - m1) - xh[k][e] * m2) * rs);
        dxr[i] = o;
      }
    }
  }
  if (*abort_flag != 0u && t == 0)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  __syncthreads();
  float* pdg = partial + static_cast<size_t>(blockIdx.x) * 2 * D;
  float* pdb = pdg + D;
#pragma unroll
  for (int k = 0; k < kMaxV; ++k) {
    const int i = t + k * kThreads;
    if (i < nvec) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) { pdg[i * VEC + e] = dg[k][e]; pdb[i * VEC + e] = db[k][e]; }
    }
  }
}

// softmax of rows too long for registers but not for shared memory (up to 220 KB, e.g. a 50304-entry f32
// vocabulary row): one 1024-thread CTA per SM stages its row in shared memory while it takes the running
// max / sum (four 16-byte loads in flight per thread), then normalises out of shared memory.  HBM sees the row
// once in each direction; the two-pass kernel re-read it from HBM because the rows in flight plus their
// outputs do not fit L2 (measured 4.1 GB read for a 1.65 GB input).
constexpr int kSmemRowThreads = 1024;
constexpr int kSmemRowBytes = 220 * 1024;

template <typename T, int VEC>
__global__ void __launch_bounds__(kSmemRowThreads)
softmax_smem_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t D, float* __restrict__ row_stats) {
  extern __shared__ uint4 row_smem_raw[];
  __shared__ float red[kSmemRowThreads / 32];
  using P = Pack<T, VEC>;
  P* sm = reinterpret_cast<P*>(row_smem_raw);
  const int nvec = D / VEC;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  constexpr int kU = 4;
  auto block_reduce = [&](float v, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();  // the previous reduction's readers are done with red
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const float r = red[lane];  // 32 warps
    return is_max ? warp_max(r) : warp_sum(r);
  };
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const P* xr = reinterpret_cast<const P*>(x + row * D);
    P* yr = reinterpret_cast<P*>(y + row * D);
    float m = -INFINITY, s = 0.0f;
    for (int i0 = t; i0 < nvec; i0 += kSmemRowThreads * kU) {
      P pks[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (i0 + u * kSmemRowThreads < nvec) pks[u] = xr[i0 + u * kSmemRowThreads];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int i = i0 + u * kSmemRowThreads;
        if (i >= nvec) break;
        sm[i] = pks[u];  // read back by this same thread below: no barrier needed for the staging itself
        float vm = ld_f32<T>(pks[u].e[0]);
#pragma unroll
        for (int e = 1; e < VEC; ++e) vm = fmaxf(vm, ld_f32<T>(pks[u].e[e]));
        if (vm > m) { s *= __expf(m - vm); m = vm; }
#pragma unroll
        for (int e = 0; e < VEC; ++e) s += __expf(ld_f32<T>(pks[u].e[e]) - m);
      }
    }
    const float row_max = block_reduce(m, true);
    const float total = block_reduce(m == -INFINITY ? 0.0f : s * __expf(m - row_max), false);
    if (row_stats != nullptr && t == 0) { row_stats[2 * row] = row_max; row_stats[2 * row + 1] = total; }
    const float recip = 1.0f / fmaxf(total, 1.0e-7f);
    for (int i = t; i < nvec; i += kSmemRowThreads) {
      const P in = sm[i];
      P o;
#pragma unroll
      for (int e = 0; e < VEC; ++e) o.e[e] = st_f32<T>(__expf(ld_f32<T>(in.e[e]) - row_max) * recip);
      yr[i] = o;
    }
  }
}

// softmax of vocabulary-sized rows (up to 224 KB): the row lives in shared memory, filled in 16 KB chunks by bulk copies
// (cp.async.bulk, completion counted per chunk on an mbarrier); thread t owns vector t of every chunk.
//   pass A  waits for the chunks as they land and takes the maximum;
//   pass B  e = exp(x - max), summed; fp32 rows keep e in place of x (one evaluation per element); the first four chunks
//           move to registers and are handed back at once;
//   pass C  writes e / sum and hands the other chunks back (a barrier the 32 warps arrive on); thread 0 refills every
//           chunk that has been handed back with the same chunk of the CTA's NEXT row.
// So the next row streams in while this one is still being summed and written: the SM reads and writes at the same time
// instead of alternating a load phase, two reductions and a store phase.  All waits are bounded; a wait that gives up raises the
// CTA's abort flag, which every thread tests after the row's first reduction barrier.
constexpr int kStreamChunkBytes = 16384;
constexpr int kStreamMaxChunks = 14;
constexpr uint32_t kStatusSoftmaxStreamWait = 0x202;

template <typename T>
__global__ void __launch_bounds__(kSmemRowThreads)
softmax_stream_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t D, float* __restrict__ row_stats,
                      uint32_t* status) {
  extern __shared__ __align__(128) uint8_t stream_row[];
  __shared__ __align__(8) uint64_t full[kStreamMaxChunks];
  __shared__ __align__(8) uint64_t consumed[kStreamMaxChunks];
  __shared__ float red[2][kSmemRowThreads / 32];
  __shared__ uint32_t abort_smem;
  volatile uint32_t* abort_flag = &abort_smem;
  constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  constexpr bool kKeepExp = sizeof(T) == 4;
  constexpr int kRegChunks = 4;   // 16 registers per thread
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int nvec = D / VEC;
  const uint32_t row_bytes = static_cast<uint32_t>(D) * sizeof(T);
  const int nchunks = (row_bytes + kStreamChunkBytes - 1) / kStreamChunkBytes;
  auto chunk_bytes = [&](int c) { return c + 1 < nchunks ? static_cast<uint32_t>(kStreamChunkBytes) : row_bytes - static_cast<uint32_t>(c) * kStreamChunkBytes; };
  if (t == 0) {
    for (int c = 0; c < nchunks; ++c) {
      mbar_init(smem_u32(&full[c]), 1);
      mbar_init(smem_u32(&consumed[c]), kSmemRowThreads / 32);
    }
    abort_smem = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  auto fill = [&](int64_t row, int c) {  // thread 0 only
    mbar_arrive_expect_tx(smem_u32(&full[c]), chunk_bytes(c));
    bulk_load(smem_u32(stream_row + static_cast<size_t>(c) * kStreamChunkBytes),
              reinterpret_cast<const uint8_t*>(x + row * D) + static_cast<size_t>(c) * kStreamChunkBytes, chunk_bytes(c),
              smem_u32(&full[c]));
  };
  // one polling lane per warp; gives up when the limit is reached or another thread already has
  auto wait_on = [&](uint64_t* bar, uint32_t parity) {
    if (lane == 0) {
      bool done = false;
      for (uint32_t spin = 0; spin < kRingSpinLimit && !done; ++spin) {
        done = mbar_try_wait(smem_u32(bar), parity);
        if (!done && (spin & 1023u) == 1023u && *abort_flag != 0u) break;
      }
      if (!done) {
        *abort_flag = 1u;
        atomicCAS(status, 0u, kStatusSoftmaxStreamWait);
      }
    }
    __syncwarp();
  };
  uint32_t red_phase = 0;
  auto block_reduce = [&](float v, bool is_max) {  // one barrier: the exchange buffer alternates between calls
    v = is_max ? warp_max(v) : warp_sum(v);
    float* buf = red[red_phase & 1u];
    ++red_phase;
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    const float r = buf[lane];  // 32 warps
    return is_max ? warp_max(r) : warp_sum(r);
  };
  if (t == 0 && blockIdx.x < rows)
    for (int c = 0; c < nchunks; ++c) fill(blockIdx.x, c);
  const float2 log2e = splat2(1.4426950408889634f);
  uint32_t it = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const uint32_t ph = it & 1u;
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
    // ---- pass A
    float m = -INFINITY;
    for (int c = 0; c < nchunks; ++c) {
      wait_on(&full[c], ph);
      const int i = c * (kStreamChunkBytes / 16) + t;
      if (i < nvec) {
        const uint4 v = reinterpret_cast<const uint4*>(stream_row)[i];
        for_pairs<T>(v, [&](int, float2 f) { m = fmaxf(m, fmaxf(f.x, f.y)); });
      }
    }
    const float row_max = block_reduce(m, true);
    if (*abort_flag != 0u) break;  // raised before that barrier by whoever gave up: uniform
    // ---- pass B
    const float2 neg_max = splat2(-row_max);
    const int64_t next = row + gridDim.x;
    int refill = 0;  // thread 0: chunks of the next row requested so far
    auto hand_back = [&](int c) {   // every lane is done with chunk c of this row
      if (next >= rows) return;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&consumed[c]));
      // thread 0 refills whatever the 32 warps have handed back so far, without waiting: a producer that blocked here
      // would fall a chunk further behind the other warps at every step and delay the whole next row
      if (t == 0)
        while (refill < c && mbar_test_wait(smem_u32(&consumed[refill]), ph)) fill(next, refill++);
    };
    auto exp_of = [&](float2 f) {
      const float2 a = __fmul2_rn(__fadd2_rn(f, neg_max), log2e);
      float2 e;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(a.x));
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(a.y));
      return e;
    };
    float2 acc = make_float2(0.0f, 0.0f);
    // The first kRegChunks chunks leave shared memory here: their e (fp32 rows) or x (16-bit rows) stays in registers
    // for pass C, so they are handed back at once and the next row's copies run during this pass and the reduction
    // after it, when the SM would otherwise move no bytes at all.  (Measured on [8192, 50304] f32: four chunks 667 us,
    // six 670, eight 702, none 707.)
    uint4 kept[kRegChunks];
#pragma unroll
    for (int c = 0; c < kRegChunks; ++c) {
      if (c < nchunks) {
        const int i = c * (kStreamChunkBytes / 16) + t;
        kept[c] = make_uint4(0u, 0u, 0u, 0u);
        if (i < nvec) {
          const uint4 v = reinterpret_cast<const uint4*>(stream_row)[i];
          uint32_t w[4];
          for_pairs<T>(v, [&](int p, float2 f) {
            const float2 e = exp_of(f);
            acc = __fadd2_rn(acc, e);
            if (kKeepExp) put_pair<T>(w, p, e);
          });
          kept[c] = kKeepExp ? make_uint4(w[0], w[1], w[2], w[3]) : v;
        }
        hand_back(c);
      }
    }
    for (int c = kRegChunks; c < nchunks; ++c) {
      const int i = c * (kStreamChunkBytes / 16) + t;
      if (i < nvec) {
        const uint4 v = reinterpret_cast<const uint4*>(stream_row)[i];
        uint32_t w[4];
        for_pairs<T>(v, [&](int p, float2 f) {
          const float2 e = exp_of(f);
          acc = __fadd2_rn(acc, e);
          if (kKeepExp) put_pair<T>(w, p, e);
        });
        if (kKeepExp) reinterpret_cast<uint4*>(stream_row)[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    // this thread's writes of e (the only generic-proxy writes to the row) are ordered before the bulk copies that will
    // refill those chunks: once per row, ahead of the barrier below and of every hand-back in pass C
    if (kKeepExp) fence_proxy_async_smem();
    const float total = block_reduce(acc.x + acc.y, false);
    if (row_stats != nullptr && t == 0) { row_stats[2 * row] = row_max; row_stats[2 * row + 1] = total; }
    const float2 recip = splat2(1.0f / fmaxf(total, 1.0e-7f));
    // ---- pass C
    auto emit = [&](int i, const uint4& v) {
      uint32_t w[4];
      for_pairs<T>(v, [&](int p, float2 f) { put_pair<T>(w, p, __fmul2_rn(kKeepExp ? f : exp_of(f), recip)); });
      yr[i] = make_uint4(w[0], w[1], w[2], w[3]);
    };
#pragma unroll
    for (int c = 0; c < kRegChunks; ++c) {
      const int i = c * (kStreamChunkBytes / 16) + t;
      if (c < nchunks && i < nvec) emit(i, kept[c]);
    }
    for (int c = kRegChunks; c < nchunks; ++c) {
      const int i = c * (kStreamChunkBytes / 16) + t;
      if (i < nvec) emit(i, reinterpret_cast<const uint4*>(stream_row)[i]);
      hand_back(c);
    }
    if (next < rows && warp == 0) {   // the rest, in order, now waiting (the other warps are at most a chunk away)
      for (int c = __shfl_sync(0xffffffffu, refill, 0); c < nchunks; ++c) {
        wait_on(&consumed[c], ph);
        if (t == 0 && *abort_flag == 0u) fill(next, c);
      }
    }
  }
  if (*abort_flag != 0u && t == 0)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let copies still in flight land before the CTA's memory is reused
  __syncthreads();
}

template <typename T, int VEC, int kMode>
int32_t launch_row_kernel(const void* x, const void* gamma, const void* beta, void* y, void* mean_sum, void* rstd,
                          int64_t rows, int64_t D, int sm_count, cudaStream_t st, float* stats, uint32_t* status) {
  const T* xp = static_cast<const T*>(x);
  const T* gp = static_cast<const T*>(gamma);
  const T* bp = static_cast<const T*>(beta);
  T* yp = static_cast<T*>(y);
  T* mp = static_cast<T*>(mean_sum);
  T* rp = static_cast<T*>(rstd);
  const int d = static_cast<int>(D);
  const int64_t nvec = D / VEC;
  // Measured on B200: rows handled by one warp (no CTA-wide barrier) run best as many short-lived CTAs;
  // rows that need the whole CTA run best as persistent CTAs that prefetch their next row into L2.
  // `resident`: CTAs of the chosen instance that fit on one SM.  A persistent grid larger than sm_count * resident
  // runs as one full wave plus a tail wave that starts late and walks as many rows per CTA.
  auto launch_grid = [&](int tpr, int max_v, int resident) {
    const int64_t ctas = (rows * tpr + kRowThreads - 1) / kRowThreads;
    int64_t cap = static_cast<int64_t>(sm_count) * (tpr == 32 ? 32 : std::max(1, std::min(resident, 8)));
    if (max_v == 0) {
      // rows too long for registers are read twice: keep the rows in flight within ~64 MB so that the second
      // read finds them in L2 (126 MB) instead of HBM
      const int64_t row_bytes = D * static_cast<int64_t>(sizeof(T));
      cap = std::max<int64_t>(sm_count, std::min<int64_t>(cap, (64ll << 20) / std::max<int64_t>(row_bytes, 1)));
    }
    return static_cast<int>(ctas < cap ? ctas : cap);
  };
#define NOVA_ROW(TPR_, MAXV_)                                                                                        \
  do {                                                                                                               \
    static int resident_ = 0; /* same on every device this library runs on (one architecture) */                     \
    if (resident_ == 0 &&                                                                                            \
        (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_, row_kernel<T, VEC, TPR_, MAXV_, kMode>, kRowThreads, 0) != \
             cudaSuccess || resident_ <= 0)) {                                                                       \
      cudaGetLastError();                                                                                            \
      resident_ = 4;                                                                                                 \
    }                                                                                                                \
    row_kernel<T, VEC, TPR_, MAXV_, kMode><<<launch_grid(TPR_, MAXV_, resident_), kRowThreads, 0, st>>>(             \
        xp, gp, bp, yp, mp, rp, rows, d, (TPR_) == 32 ? 0 : 1, stats);                                               \
  } while (0)
  // Vectors a thread keeps in registers are kept few (occupancy sets the bytes in flight per SM):
  // longer rows get more threads, not more registers.
  constexpr int kWarpMv = VEC == 1 ? 32 : (kMode == 0 ? 4 : 8);
  // layer_norm rows of 2 KB .. 32 KB: the shared-memory ring (bulk copies, one barrier per row)
  if (kMode == 0 && VEC > 1 && status != nullptr && nvec > 32 * kWarpMv && nvec <= kRowThreads * 8 && ring_rows_enabled()) {
    const size_t row_bytes = static_cast<size_t>(D) * sizeof(T);
    // Two slots per CTA: one row landing while one is reduced.  With four CTAs per SM that already keeps HBM busy, and
    // deeper rings measured SLOWER on [8192, 4096] bf16 (2 slots 5.05 TB/s, 4: 4.87, 6: 4.53): more rows in flight
    // from every SM scatter the DRAM accesses.
    int stages = 2;
    if (const int64_t o = options().ring_stages.load(); o >= 2 && o <= kRingMaxStages) stages = static_cast<int>(o);
#define NOVA_LN_RING(MAXV_)                                                                                          \
    do {                                                                                                             \
      auto kernel = ln_ring_kernel<T, MAXV_>;                                                                        \
      const size_t smem = stages * row_bytes;                                                                        \
      int resident = ring_resident_ctas(kernel, kRowThreads, smem);                                                  \
      if (resident <= 0) return fail(NOVA_B200_ERR_CUDA, std::string("layer_norm: the ring kernel cannot be configured: ") + nova_b200_last_error_string()); \
      if (const int64_t o = options().ring_ctas.load(); o >= 1 && o < resident) resident = static_cast<int>(o);      \
      const int grid = static_cast<int>(std::min<int64_t>(rows, static_cast<int64_t>(sm_count) * resident));         \
      kernel<<<grid, kRowThreads, smem, st>>>(xp, gp, bp, yp, mp, rp, rows, d, stages, status);                      \
    } while (0)
    if (nvec <= kRowThreads * 2) NOVA_LN_RING(2);
    else if (nvec <= kRowThreads * 4) NOVA_LN_RING(4);
    else NOVA_LN_RING(8);
#undef NOVA_LN_RING
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }
  if (kMode == 0 && VEC > 1 && nvec <= 32 * 4 && ring_rows_enabled()) {
    // one warp per row, many short-lived CTAs (see the note on launch_grid)
    const int64_t ctas = (rows + kRowThreads / 32 - 1) / (kRowThreads / 32);
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(ctas, static_cast<int64_t>(sm_count) * 32)));
    if (nvec <= 32) ln_warp_kernel<T, 1><<<grid, kRowThreads, 0, st>>>(xp, gp, bp, yp, mp, rp, rows, d);
    else if (nvec <= 64) ln_warp_kernel<T, 2><<<grid, kRowThreads, 0, st>>>(xp, gp, bp, yp, mp, rp, rows, d);
    else ln_warp_kernel<T, 4><<<grid, kRowThreads, 0, st>>>(xp, gp, bp, yp, mp, rp, rows, d);
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }
  if (kMode == 1 && VEC > 1 && nvec <= 32 * 8 && ring_rows_enabled()) {
    // one warp per row, many short-lived CTAs (see the note on launch_grid)
    const int64_t ctas = (rows + kRowThreads / 32 - 1) / (kRowThreads / 32);
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(ctas, static_cast<int64_t>(sm_count) * 32)));
    if (nvec <= 32 * 2) softmax_warp_kernel<T, 2><<<grid, kRowThreads, 0, st>>>(xp, yp, rows, d, stats);
    else if (nvec <= 32 * 4) softmax_warp_kernel<T, 4><<<grid, kRowThreads, 0, st>>>(xp, yp, rows, d, stats);
    else softmax_warp_kernel<T, 8><<<grid, kRowThreads, 0, st>>>(xp, yp, rows, d, stats);
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }
  if (kMode == 1 && VEC > 1 && status != nullptr && nvec > 32 * 8 && nvec <= kRowThreads * 8 && ring_rows_enabled()) {
    const size_t row_bytes = static_cast<size_t>(D) * sizeof(T);
    int stages = 2;
    if (const int64_t o = options().ring_stages.load(); o >= 2 && o <= kRingMaxStages) stages = static_cast<int>(o);
    // CTAs per SM, measured (fraction of the copy bandwidth with 2 / 3 / 4 resident): rows of 8 KB 0.68 / 0.84 / 0.80,
    // of 16 KB 0.97 / 0.83 / 0.81 (f16) and 0.91 / 0.87 / 0.87 (f32), of 32 KB 0.83 / 0.79 / -: more rows in flight
    // than that only scatter the DRAM accesses
    const int best_ctas = row_bytes <= (8u << 10) ? 3 : 2;
#define NOVA_SM_RING(MAXV_)                                                                                          \
    do {                                                                                                             \
      auto kernel = softmax_ring_kernel<T, MAXV_>;                                                                   \
      const size_t smem = stages * row_bytes;                                                                        \
      int resident = ring_resident_ctas(kernel, kRowThreads, smem);                                                  \
      if (resident <= 0) return fail(NOVA_B200_ERR_CUDA, std::string("softmax: the ring kernel cannot be configured: ") + nova_b200_last_error_string()); \
      if (const int64_t o = options().ring_ctas.load(); o >= 1) resident = std::min(resident, static_cast<int>(o));  \
      else resident = std::min(resident, best_ctas);                                                                 \
      const int grid = static_cast<int>(std::min<int64_t>(rows, static_cast<int64_t>(sm_count) * resident));         \
      kernel<<<grid, kRowThreads, smem, st>>>(xp, yp, rows, d, stages, stats, status);                               \
    } while (0)
    if (nvec <= kRowThreads * 2) NOVA_SM_RING(2);
    else if (nvec <= kRowThreads * 4) NOVA_SM_RING(4);
    else NOVA_SM_RING(8);
#undef NOVA_SM_RING
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }
  if (VEC == 1) {
    // scalar path (row length or base not 16-byte friendly)
    if (nvec <= 32 * kWarpMv) NOVA_ROW(32, kWarpMv);
    else if (nvec <= kRowThreads * kWarpMv) NOVA_ROW(kRowThreads, kWarpMv);
    else NOVA_ROW(kRowThreads, 0);
  } else {
    if (nvec <= 32 * 2) NOVA_ROW(32, 2);
    else if (nvec <= 32 * 4) NOVA_ROW(32, 4);
    else if (nvec <= 32 * kWarpMv) NOVA_ROW(32, kWarpMv);
    else if (nvec <= kRowThreads * 2) NOVA_ROW(kRowThreads, 2);
    else if (nvec <= kRowThreads * 4) NOVA_ROW(kRowThreads, 4);
    else if (nvec <= kRowThreads * 8) NOVA_ROW(kRowThreads, 8);
    else if (nvec <= kRowThreads * 16) NOVA_ROW(kRowThreads, 16);
    else if (kMode == 1 && status != nullptr && ring_rows_enabled() && D * static_cast<int64_t>(sizeof(T)) <= kSmemRowBytes) {
      auto kernel = softmax_stream_kernel<T>;
      const int smem = static_cast<int>((D * sizeof(T) + kStreamChunkBytes - 1) / kStreamChunkBytes) * kStreamChunkBytes;
      static thread_local int configured_device = -1;  // (a function attribute belongs to one device's copy of the kernel)
      int device = 0;
      NOVA_CUDA_OK(cudaGetDevice(&device));
      if (configured_device != device) {
        NOVA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamMaxChunks * kStreamChunkBytes));
        configured_device = device;
      }
      const int grid = static_cast<int>(rows < sm_count ? rows : sm_count);
      kernel<<<grid, kSmemRowThreads, smem, st>>>(xp, yp, rows, d, stats, status);
    } else if (kMode == 1 && D * static_cast<int64_t>(sizeof(T)) <= kSmemRowBytes) {
      auto kernel = softmax_smem_kernel<T, VEC>;
      const int smem = static_cast<int>(D * sizeof(T));
      NOVA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemRowBytes));
      const int grid = static_cast<int>(rows < sm_count ? rows : sm_count);
      kernel<<<grid, kSmemRowThreads, smem, st>>>(xp, yp, rows, d, stats);
    } else NOVA_ROW(kRowThreads, 0);
  }
#undef NOVA_ROW
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

template <int kMode>
int32_t dispatch_row_kernel(const void* x, const void* gamma, const void* beta, void* y, void* mean_sum, void* rstd,
                            int64_t rows, int64_t D, int32_t dtype, int sm_count, cudaStream_t st, float* stats = nullptr,
                            uint32_t* status = nullptr) {
  const int es = dtype_bytes(dtype);
  const int vec = 16 / es;
  auto aligned16 = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec_ok = D % vec == 0 && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
  switch (dtype) {
    case NOVA_B200_F32:
      return vec_ok ? launch_row_kernel<float, 4, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status)
                    : launch_row_kernel<float, 1, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status);
    case NOVA_B200_F16:
      return vec_ok ? launch_row_kernel<__half, 8, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status)
                    : launch_row_kernel<__half, 1, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status);
    case NOVA_B200_BF16:
      return vec_ok
                 ? launch_row_kernel<__nv_bfloat16, 8, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status)
                 : launch_row_kernel<__nv_bfloat16, 1, kMode>(x, gamma, beta, y, mean_sum, rstd, rows, D, sm_count, st, stats, status);
    default:
      return fail(NOVA_B200_ERR_UNSUPPORTED, "row op: dtype must be f32, f16 or bf16");
  }
}

// ---------------------------------------------------------------- gather

// A group of G = 2^g_shift threads (G <= 32, a power of two >= the units in a row when that is < 32) copies
// one output row: the group's threads take consecutive 16-byte (or W-byte) units, four in flight each.
// The row's index is read once per thread; there are no divisions on the copy path.
template <typename U>
__global__ void __launch_bounds__(256)
gather_kernel(const U* __restrict__ in, const void* __restrict__ idx, U* __restrict__ out, int64_t pre,
              int64_t axis_len, int64_t units_per_row, int64_t n_idx, int32_t idx_dtype, int32_t batched,
              int32_t g_shift, unsigned long long* bad_count) {
  constexpr int kUnroll = 4;
  const int64_t out_rows = pre * n_idx;
  const int64_t G = int64_t(1) << g_shift;
  const int64_t gthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t u0 = tid & (G - 1);
  for (int64_t orow = tid >> g_shift; orow < out_rows; orow += gthreads >> g_shift) {
    const int64_t p = n_idx == out_rows ? 0 : orow / n_idx;  // pre == 1 (embedding lookup): no division
    const int64_t q = batched ? orow : orow - p * n_idx;
    int64_t id;
    if (idx_dtype == NOVA_B200_I16) id = static_cast<int64_t>(static_cast<const uint16_t*>(idx)[q]);  // zero-extended
    else if (idx_dtype == NOVA_B200_I32) id = static_cast<int64_t>(static_cast<const int32_t*>(idx)[q]);
    else id = static_cast<const int64_t*>(idx)[q];
    const bool ok = id >= 0 && id < axis_len;
    if (!ok && u0 == 0 && bad_count) atomicAdd(bad_count, 1ull);
    const U* src = in + (p * axis_len + (ok ? id : 0)) * units_per_row;
    U* dst = out + orow * units_per_row;
    for (int64_t u = u0; u < units_per_row; u += G * kUnroll) {
      U v[kUnroll];
#pragma unroll
      for (int k = 0; k < kUnroll; ++k) {
        v[k] = U{};
        if (ok && u + k * G < units_per_row) v[k] = src[u + k * G];
      }
#pragma unroll
      for (int k = 0; k < kUnroll; ++k)
        if (u + k * G < units_per_row) dst[u + k * G] = v[k];
    }
  }
}

// ---------------------------------------------------------------- elementwise

__device__ __forceinline__ float gelu_tanh_accurate(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  return 0.5f * x * (1.0f + tanhf(u));
}

template <typename T, int VEC>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, int32_t act) {
  using P = Pack<T, VEC>;
  const int64_t nv = n / VEC;
  const P* xp = reinterpret_cast<const P*>(x);
  P* yp = reinterpret_cast<P*>(y);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    P v = xp[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float f = ld_f32<T>(v.e[e]);
      v.e[e] = st_f32<T>(act == NOVA_B200_ACT_RELU ? fmaxf(f, 0.0f)
                                                    : (act == NOVA_B200_ACT_GELU_TANH ? gelu_tanh_accurate(f) : f));
    }
    yp[i] = v;
  }
}

// 0.5(1 + tanh u) + 0.5 x (1 - tanh^2 u) u', u = 0.79788456 (x + 0.044715 x^3)
__device__ __forceinline__ float gelu_tanh_grad_accurate(float x) {
  const float x2 = x * x;
  const float t = tanhf(0.7978845608028654f * fmaf(0.044715f * x, x2, x));
  const float du = 0.7978845608028654f * fmaf(0.134145f, x2, 1.0f);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
}

template <typename T, int VEC>
__global__ void gelu_backward_kernel(const T* __restrict__ go, const T* __restrict__ x, T* __restrict__ y, int64_t n) {
  using P = Pack<T, VEC>;
  const int64_t nv = n / VEC;
  const P* gp = reinterpret_cast<const P*>(go);
  const P* xp = reinterpret_cast<const P*>(x);
  P* yp = reinterpret_cast<P*>(y);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const P g = gp[i];
    P v = xp[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v.e[e] = st_f32<T>(ld_f32<T>(g.e[e]) * gelu_tanh_grad_accurate(ld_f32<T>(v.e[e])));
    yp[i] = v;
  }
}

template <typename T, int VEC>
__global__ void add_rowbcast_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows,
                                    int64_t cols, int32_t b_is_full) {
  using P = Pack<T, VEC>;
  const int64_t cv = cols / VEC;
  const int64_t nv = rows * cv;
  const P* ap = reinterpret_cast<const P*>(a);
  const P* bp = reinterpret_cast<const P*>(b);
  P* op = reinterpret_cast<P*>(out);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const P va = ap[i];
    const P vb = bp[b_is_full ? i : i % cv];
    P o;
#pragma unroll
    for (int e = 0; e < VEC; ++e) o.e[e] = st_f32<T>(ld_f32<T>(va.e[e]) + ld_f32<T>(vb.e[e]));
    op[i] = o;
  }
}

// out = a (op) b with numpy-style broadcasting over up to six dims: every operand carries one element stride per
// output dim, 0 where it broadcasts.  The launcher collapses dims first, so the common shapes (equal shapes, a
// bias along the rows, one scalar, a batch of equal slices) arrive as at most two dims with unit or zero strides
// and the index arithmetic is one division per element; only odd broadcasts walk all six.
struct BinaryDims {
  int32_t rank;
  int64_t shape[6], sa[6], sb[6];
};

template <typename T, int kOp>
__global__ void binary_broadcast_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n,
                                        BinaryDims d) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, oa = 0, ob = 0;
#pragma unroll 1
    for (int k = d.rank - 1; k > 0; --k) {
      const int64_t q = rem / d.shape[k], r = rem - q * d.shape[k];
      oa += r * d.sa[k];
      ob += r * d.sb[k];
      rem = q;
    }
    oa += rem * d.sa[0];
    ob += rem * d.sb[0];
    const float x = ld_f32<T>(a[oa]), y = ld_f32<T>(b[ob]);
    out[i] = st_f32<T>(kOp == 0 ? x + y : (kOp == 1 ? x - y : x * y));
  }
}

// Column sums of x[rows, cols] (the bias gradient of nova.linear_backward).  Pass 1: CTA (cx, ry) owns 64
// columns and every gridDim.y-th block of 32 rows; a warp reads one row segment of 64 columns (128 B of
// 16-bit data) per step, so loads are coalesced, and accumulates in fp32; the 8 warps' partials meet in shared
// memory and one partial row per CTA goes to partial[ry, cols].  Pass 2 adds the gridDim.y partial rows.
template <typename T>
__global__ void __launch_bounds__(256)
column_sum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, int64_t rows, int64_t cols) {
  __shared__ float red[8][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 64 + lane * 2;
  float s0 = 0.0f, s1 = 0.0f;
  for (int64_t r = static_cast<int64_t>(blockIdx.y) * 8 + warp; r < rows; r += static_cast<int64_t>(gridDim.y) * 8) {
    const T* row = x + r * cols;
    if (c0 < cols) s0 += ld_f32<T>(row[c0]);
    if (c0 + 1 < cols) s1 += ld_f32<T>(row[c0 + 1]);
  }
  red[warp][lane * 2] = s0;
  red[warp][lane * 2 + 1] = s1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 64 + threadIdx.x;
    if (c < cols) partial[static_cast<int64_t>(blockIdx.y) * cols + c] = t;
  }
}

template <typename T>
__global__ void column_sum_final_kernel(const float* __restrict__ partial, T* __restrict__ out, int64_t cols, int splits) {
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < cols;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float t = 0.0f;
    for (int k = 0; k < splits; ++k) t += partial[static_cast<int64_t>(k) * cols + c];
    out[c] = st_f32<T>(t);
  }
}

// layer_norm_backward.  One CTA walks rows r = blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns the same
// vectors (t, t + blockDim.x, ...) of every row, so the per-column sums for dgamma / dbeta accumulate in its
// registers over all the CTA's rows while dx is produced from the same single read of gy and x.  Per row:
//   mean = mean_sum/D, xhat = (x - mean) rstd, gyg = gy gamma, s1 = sum gyg, s2 = sum gyg xhat (one block
//   reduction of the pair), dx = ((gyg - s1/D) - xhat s2/D) rstd.
// The CTA's column sums go to partial[blockIdx.x][0|1][D] (fp32); ln_backward_finish_kernel adds them up.
// HBM traffic: gy, x read once, dx written once (+ the small partials).
template <typename T, int VEC, int kMaxV, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
ln_backward_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ gamma,
                   const T* __restrict__ mean_sum, const T* __restrict__ rstd, T* __restrict__ dx,
                   float* __restrict__ partial, int64_t rows, int32_t D) {
  __shared__ float red[2][kMaxThreads / 32];
  using P = Pack<T, VEC>;
  const int nvec = D / VEC;
  const int nthreads = blockDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = nthreads >> 5;
  const float inv_d = 1.0f / static_cast<float>(D);
  P gam[kMaxV];
  float dg[kMaxV][VEC], db[kMaxV][VEC];
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) {
    const int v = threadIdx.x + i * nthreads;
    if (v < nvec) gam[i] = reinterpret_cast<const P*>(gamma)[v];
#pragma unroll
    for (int e = 0; e < VEC; ++e) dg[i][e] = db[i][e] = 0.0f;
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const P* gyr = reinterpret_cast<const P*>(gy + r * D);
    const P* xr = reinterpret_cast<const P*>(x + r * D);
    if (r + gridDim.x < rows) {  // the CTA's next row on its way into L2 while this one is reduced and stored
      constexpr int kVecPerLine = 128 / static_cast<int>(sizeof(P));
      const P* ng = reinterpret_cast<const P*>(gy + (r + gridDim.x) * D);
      const P* nx = reinterpret_cast<const P*>(x + (r + gridDim.x) * D);
      for (int i = threadIdx.x * kVecPerLine; i < nvec; i += nthreads * kVecPerLine) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(ng + i));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + i));
      }
    }
    P pg[kMaxV], px[kMaxV];
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = threadIdx.x + i * nthreads;
      if (v < nvec) { pg[i] = gyr[v]; px[i] = xr[v]; }
    }
    const float mean = ld_f32<T>(mean_sum[r]) * inv_d;
    const float rs = ld_f32<T>(rstd[r]);
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      if (threadIdx.x + i * nthreads < nvec) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float g = ld_f32<T>(pg[i].e[e]);
          const float xhat = (ld_f32<T>(px[i].e[e]) - mean) * rs;
          const float gyg = g * ld_f32<T>(gam[i].e[e]);
          s1 += gyg;
          s2 = fmaf(gyg, xhat, s2);
          dg[i][e] = fmaf(g, xhat, dg[i][e]);
          db[i][e] += g;
        }
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (nwarps > 1) {
      __syncthreads();  // the previous row's readers are done with red
      if (lane == 0) { red[0][warp] = s1; red[1][warp] = s2; }
      __syncthreads();
      s1 = warp_sum(lane < nwarps ? red[0][lane] : 0.0f);
      s2 = warp_sum(lane < nwarps ? red[1][lane] : 0.0f);
    }
    const float m1 = s1 * inv_d, m2 = s2 * inv_d;
    P* dxr = reinterpret_cast<P*>(dx + r * D);
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = threadIdx.x + i * nthreads;
      if (v < nvec) {
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float xhat = (ld_f32<T>(px[i].e[e]) - mean) * rs;
          const float gyg = ld_f32<T>(pg[i].e[e]) * ld_f32<T>(gam[i].e[e]);
          o.e[e] = st_f32<T>(((gyg - m1) - xhat * m2) * rs);
        }
        dxr[v] = o;
      }
    }
  }
  float* pdg = partial + static_cast<size_t>(blockIdx.x) * 2 * D;
  float* pdb = pdg + D;
#pragma unroll
  for (int i = 0; i < kMaxV; ++i) {
    const int v = threadIdx.x + i * nthreads;
    if (v < nvec) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) { pdg[v * VEC + e] = dg[i][e]; pdb[v * VEC + e] = db[i][e]; }
    }
  }
}

// The same for rows of at most kMaxThreads vectors, kRowsPer rows per trip: one vector per thread and row, all
// 2 * kRowsPer loads of a trip issued before the first is used and ONE block reduction for the trip's
// 2 * kRowsPer sums, so the per-row latency chain (load, shuffle tree, two barriers, store) is paid once per
// kRowsPer rows.
template <typename T, int VEC, int kRowsPer, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
ln_backward_rows_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ gamma,
                        const T* __restrict__ mean_sum, const T* __restrict__ rstd, T* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows, int32_t D) {
  __shared__ float red[2][2 * kRowsPer][kMaxThreads / 32];  // exchange buffer, alternating per trip: one barrier per trip
  uint32_t trip = 0;
  using P = Pack<T, VEC>;
  const int nvec = D / VEC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const bool mine = static_cast<int>(threadIdx.x) < nvec;
  const float inv_d = 1.0f / static_cast<float>(D);
  P gam;
  float dg[VEC], db[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) { dg[e] = db[e] = 0.0f; gam.e[e] = st_f32<T>(0.0f); }
  if (mine) gam = reinterpret_cast<const P*>(gamma)[threadIdx.x];
  const int64_t step = static_cast<int64_t>(gridDim.x) * kRowsPer;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * kRowsPer; r0 < rows; r0 += step) {
    P pg[kRowsPer], px[kRowsPer];
    float mean[kRowsPer], rs[kRowsPer], s[2 * kRowsPer];
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const int64_t r = r0 + k;
      if (mine && r < rows) {
        pg[k] = reinterpret_cast<const P*>(gy + r * D)[threadIdx.x];
        px[k] = reinterpret_cast<const P*>(x + r * D)[threadIdx.x];
      }
    }
    if (mine && (threadIdx.x * sizeof(P)) % 128 == 0) {  // the trip after this one, one request per 128-byte line
#pragma unroll
      for (int k = 0; k < kRowsPer; ++k) {
        const int64_t r = r0 + step + k;
        if (r < rows) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const P*>(gy + r * D) + threadIdx.x));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const P*>(x + r * D) + threadIdx.x));
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const int64_t r = r0 + k;
      const bool live = r < rows;
      mean[k] = live ? ld_f32<T>(mean_sum[r]) * inv_d : 0.0f;
      rs[k] = live ? ld_f32<T>(rstd[r]) : 0.0f;
      float s1 = 0.0f, s2 = 0.0f;
      if (mine && live) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float g = ld_f32<T>(pg[k].e[e]);
          const float xhat = (ld_f32<T>(px[k].e[e]) - mean[k]) * rs[k];
          const float gyg = g * ld_f32<T>(gam.e[e]);
          s1 += gyg;
          s2 = fmaf(gyg, xhat, s2);
          dg[e] = fmaf(g, xhat, dg[e]);
          db[e] += g;
        }
      }
      s[2 * k] = warp_sum(s1);
      s[2 * k + 1] = warp_sum(s2);
    }
    if (nwarps > 1) {
      // (a warp writes this buffer again two trips on, after the barrier of the trip in between: by then every
      // reader of this trip is done)
      float (*buf)[kMaxThreads / 32] = red[trip & 1u];
      ++trip;
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < 2 * kRowsPer; ++j) buf[j][warp] = s[j];
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 2 * kRowsPer; ++j) s[j] = warp_sum(lane < nwarps ? buf[j][lane] : 0.0f);
    }
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const int64_t r = r0 + k;
      if (mine && r < rows) {
        const float m1 = s[2 * k] * inv_d, m2 = s[2 * k + 1] * inv_d;
        const P qg = pg[k], qx = px[k];  // (re-reading them from L1 to free registers was measured: slower)
        P o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float xhat = (ld_f32<T>(qx.e[e]) - mean[k]) * rs[k];
          const float gyg = ld_f32<T>(qg.e[e]) * ld_f32<T>(gam.e[e]);
          o.e[e] = st_f32<T>(((gyg - m1) - xhat * m2) * rs[k]);
        }
        reinterpret_cast<P*>(dx + r * D)[threadIdx.x] = o;
      }
    }
  }
  if (mine) {
    float* pdg = partial + static_cast<size_t>(blockIdx.x) * 2 * D;
    float* pdb = pdg + D;
#pragma unroll
    for (int e = 0; e < VEC; ++e) { pdg[threadIdx.x * VEC + e] = dg[e]; pdb[threadIdx.x * VEC + e] = db[e]; }
  }
}

// layer_norm_backward for rows of one 16-byte vector per thread (at most kThreads vectors), kRowsPer rows per trip,
// in packed fp32 arithmetic.  Per trip: 2 kRowsPer vector loads in flight, the first half of the arithmetic
//   xhat = x rstd - mean rstd,  gg = gy gamma,  s1 += gg,  s2 += gg xhat,  dgamma += gy xhat,  dbeta += gy
// (six packed operations per element pair), ONE exchange of the 2 kRowsPer row sums (shuffle tree that halves the
// carried values, one shared-memory round, one barrier), then dx = gg rstd - xhat (s2/D) rstd - (s1/D) rstd as two
// packed fmas from the xhat and gg kept in registers.  Rows past the end and threads past the row load zeros and so
// add nothing anywhere.
template <typename T, int kRowsPer, int kThreads, int kMinCtas>
__global__ void __launch_bounds__(kThreads, kMinCtas)
ln_backward_packed_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ gamma,
                          const T* __restrict__ mean_sum, const T* __restrict__ rstd, T* __restrict__ dx,
                          float* __restrict__ partial, int64_t rows, int32_t D) {
  constexpr int VEC = 16 / static_cast<int>(sizeof(T)), NP = VEC / 2, NS = 2 * kRowsPer;
  constexpr int kSlots = kThreads > 512 ? 32 : 16;  // warps whose partials one sum collects
  constexpr int kLanesPerSum = kSlots / 4;          // lanes that each add one float4 of them
  static_assert(kThreads / 32 <= kSlots && NS * kLanesPerSum <= 32, "one float4 of warp partials per lane");
  __shared__ __align__(16) float red[2][NS][kSlots];  // [trip parity][sum][warp]; slots of absent warps stay zero
  const int nvec = D / VEC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool mine = static_cast<int>(threadIdx.x) < nvec;
  const float inv_d = 1.0f / static_cast<float>(D);
  for (int i = threadIdx.x; i < 2 * NS * kSlots; i += blockDim.x) (&red[0][0][0])[i] = 0.0f;
  __syncthreads();
  griddep_launch_dependents();  // the finish kernel may be scheduled as SMs free up; it waits for this grid's end
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const uint4 gam_raw = mine ? reinterpret_cast<const uint4*>(gamma)[threadIdx.x] : zero4;
  float2 gam[NP], dg[NP], db[NP];
  gam[0] = pair_of<T, 0>(gam_raw);
  gam[1] = pair_of<T, 1>(gam_raw);
  if constexpr (NP == 4) { gam[2] = pair_of<T, 2>(gam_raw); gam[3] = pair_of<T, 3>(gam_raw); }
#pragma unroll
  for (int p = 0; p < NP; ++p) dg[p] = db[p] = make_float2(0.0f, 0.0f);
  uint32_t trip = 0;
  // Running pointers: the row addresses of a trip are these plus k * D, and a trip advances them by one constant.  (With
  // the addresses recomputed from the row index every trip, 64-bit multiplies and the re-reading of kernel parameters
  // and thread ids they drag in were a third of all instructions executed: ncu opcode counts.)
  const int tid = threadIdx.x;
  const int64_t step = static_cast<int64_t>(gridDim.x) * kRowsPer;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kRowsPer;
  const uint4* gy_p = reinterpret_cast<const uint4*>(gy + first * D) + tid;
  const uint4* x_p = reinterpret_cast<const uint4*>(x + first * D) + tid;
  uint4* dx_p = reinterpret_cast<uint4*>(dx + first * D) + tid;
  const T* ms_p = mean_sum + first;
  const T* rs_p = rstd + first;
  const int row_vecs = D / VEC;   // vectors from one row to the next
  const int64_t trip_vecs = step * row_vecs;
  const bool prefetcher = mine && (tid & 7) == 0;
  for (int64_t r0 = first; r0 < rows; r0 += step, gy_p += trip_vecs, x_p += trip_vecs, dx_p += trip_vecs,
               ms_p += step, rs_p += step) {
    uint4 pg[kRowsPer], px[kRowsPer];
    float rs[kRowsPer], nmr[kRowsPer];
    const int live_rows = static_cast<int>(rows - r0 < kRowsPer ? rows - r0 : kRowsPer);   // uniform
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const bool live = mine && k < live_rows;
      pg[k] = live ? gy_p[k * row_vecs] : zero4;
      px[k] = live ? x_p[k * row_vecs] : zero4;
    }
    if (prefetcher) {  // the trip after this one into L2, one request per 128-byte line
      const int64_t ahead = rows - (r0 + step);
#pragma unroll
      for (int k = 0; k < kRowsPer; ++k) {
        if (k < ahead) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(gy_p + trip_vecs + k * row_vecs));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(x_p + trip_vecs + k * row_vecs));
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const bool live = k < live_rows;
      rs[k] = live ? ld_f32<T>(rs_p[k]) : 0.0f;
      nmr[k] = live ? -ld_f32<T>(ms_p[k]) * inv_d * rs[k] : 0.0f;
    }
    float2 kxh[kRowsPer][NP], kgg[kRowsPer][NP];
    float s[NS];
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      float2 s1 = make_float2(0.0f, 0.0f), s2 = make_float2(0.0f, 0.0f);
      const float2 rs2 = splat2(rs[k]), nmr2 = splat2(nmr[k]);
      auto first_half = [&](int p, float2 g2, float2 x2) {
        const float2 xh = __ffma2_rn(x2, rs2, nmr2);
        const float2 gg = __fmul2_rn(g2, gam[p]);
        s1 = __fadd2_rn(s1, gg);
        s2 = __ffma2_rn(gg, xh, s2);
        dg[p] = __ffma2_rn(g2, xh, dg[p]);
        db[p] = __fadd2_rn(db[p], g2);
        kxh[k][p] = xh;
        kgg[k][p] = gg;
      };
      first_half(0, pair_of<T, 0>(pg[k]), pair_of<T, 0>(px[k]));
      first_half(1, pair_of<T, 1>(pg[k]), pair_of<T, 1>(px[k]));
      if constexpr (NP == 4) {
        first_half(2, pair_of<T, 2>(pg[k]), pair_of<T, 2>(px[k]));
        first_half(3, pair_of<T, 3>(pg[k]), pair_of<T, 3>(px[k]));
      }
      s[2 * k] = s1.x + s1.y;
      s[2 * k + 1] = s2.x + s2.y;
    }
    // exchange: (a warp writes this buffer again two trips on, after the barrier of the trip in between: by then
    // every reader of this trip is done)
    float (*buf)[kSlots] = red[trip & 1u];
    ++trip;
    int j;
    const float mine_sum = warp_multi_sum<NS>(s, lane, j);
    if ((lane & (32 / NS - 1)) == 0) buf[j][warp] = mine_sum;
    __syncthreads();
    // lane l adds four warps' partials of sum l / kLanesPerSum; log2(kLanesPerSum) more exchanges complete it in the
    // lanes j kLanesPerSum .. (j + 1) kLanesPerSum - 1
    float4 q = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (lane < NS * kLanesPerSum) q = reinterpret_cast<const float4*>(&buf[0][0])[lane];
    float t = (q.x + q.y) + (q.z + q.w);
#pragma unroll
    for (int o = 1; o < kLanesPerSum; o <<= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
#pragma unroll
    for (int k = 0; k < kRowsPer; ++k) {
      const float m1 = __shfl_sync(0xffffffffu, t, 2 * k * kLanesPerSum) * inv_d;
      const float m2 = __shfl_sync(0xffffffffu, t, (2 * k + 1) * kLanesPerSum) * inv_d;
      const float2 a2 = splat2(rs[k]), b2 = splat2(-m2 * rs[k]), c2 = splat2(-m1 * rs[k]);
      uint4 o;
      if constexpr (NP == 4) {
        o.x = pack_pair<T>(__ffma2_rn(kxh[k][0], b2, __ffma2_rn(kgg[k][0], a2, c2)));
        o.y = pack_pair<T>(__ffma2_rn(kxh[k][1], b2, __ffma2_rn(kgg[k][1], a2, c2)));
        o.z = pack_pair<T>(__ffma2_rn(kxh[k][2], b2, __ffma2_rn(kgg[k][2], a2, c2)));
        o.w = pack_pair<T>(__ffma2_rn(kxh[k][3], b2, __ffma2_rn(kgg[k][3], a2, c2)));
      } else {
        const float2 lo = __ffma2_rn(kxh[k][0], b2, __ffma2_rn(kgg[k][0], a2, c2));
        const float2 hi = __ffma2_rn(kxh[k][1], b2, __ffma2_rn(kgg[k][1], a2, c2));
        o = make_uint4(__float_as_uint(lo.x), __float_as_uint(lo.y), __float_as_uint(hi.x), __float_as_uint(hi.y));
      }
      if (mine && k < live_rows) dx_p[k * row_vecs] = o;
    }
  }
  if (mine) {
    float* pdg = partial + static_cast<size_t>(blockIdx.x) * 2 * D + threadIdx.x * VEC;
    float* pdb = pdg + D;
#pragma unroll
    for (int p = 0; p < NP; p += 2) {
      reinterpret_cast<float4*>(pdg)[p / 2] = make_float4(dg[p].x, dg[p].y, dg[p + 1].x, dg[p + 1].y);
      reinterpret_cast<float4*>(pdb)[p / 2] = make_float4(db[p].x, db[p].y, db[p + 1].x, db[p + 1].y);
    }
  }
}

// dgamma[c] = sum over CTAs of partial[cta][0][c], dbeta[c] likewise from [cta][1][c]; several CTA slices per
// column are combined through shared memory so that short D still fills the machine.
template <typename T>
__global__ void ln_backward_finish_kernel(const float* __restrict__ partial, int32_t n_partials, int32_t D,
                                          T* __restrict__ dgamma, T* __restrict__ dbeta) {
  __shared__ float sh[2][32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;  // blockDim = (32, 32)
  griddep_wait();  // launched while the kernel that writes `partial` is still running (programmatic serialization)
  float a = 0.0f, b = 0.0f;
  if (c < D)
  {
    float a1 = 0.0f, b1 = 0.0f, a2 = 0.0f, b2 = 0.0f, a3 = 0.0f, b3 = 0.0f;
    int p = threadIdx.y;
    for (; p + 96 < n_partials; p += 128) {  // four independent loads per sum in flight
      a += partial[static_cast<size_t>(p) * 2 * D + c];
      b += partial[static_cast<size_t>(p) * 2 * D + D + c];
      a1 += partial[static_cast<size_t>(p + 32) * 2 * D + c];
      b1 += partial[static_cast<size_t>(p + 32) * 2 * D + D + c];
      a2 += partial[static_cast<size_t>(p + 64) * 2 * D + c];
      b2 += partial[static_cast<size_t>(p + 64) * 2 * D + D + c];
      a3 += partial[static_cast<size_t>(p + 96) * 2 * D + c];
      b3 += partial[static_cast<size_t>(p + 96) * 2 * D + D + c];
    }
    for (; p < n_partials; p += 32) {
      a += partial[static_cast<size_t>(p) * 2 * D + c];
      b += partial[static_cast<size_t>(p) * 2 * D + D + c];
    }
    a += a1 + a2 + a3;
    b += b1 + b2 + b3;
  }
  sh[0][threadIdx.y][threadIdx.x] = a;
  sh[1][threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && c < D) {
#pragma unroll
    for (int k = 1; k < 32; ++k) { a += sh[0][k][threadIdx.x]; b += sh[1][k][threadIdx.x]; }
    dgamma[c] = st_f32<T>(a);
    dbeta[c] = st_f32<T>(b);
  }
}

// ---------------------------------------------------------------- softmax cross-entropy, scatter_add

__device__ __forceinline__ int64_t load_index(const void* idx, int64_t q, int32_t idx_dtype) {
  if (idx_dtype == NOVA_B200_I16) return static_cast<int64_t>(static_cast<const uint16_t*>(idx)[q]);  // zero-extended
  if (idx_dtype == NOVA_B200_I32) return static_cast<int64_t>(static_cast<const int32_t*>(idx)[q]);
  return static_cast<const int64_t*>(idx)[q];
}

// loss = mean over rows of log(max(sum_exp, 1e-7)) - (x[target] - max), from the {max, sum_exp} pairs the softmax
// kernel left per row.  One CTA: every thread sums its rows in ascending order, then a fixed tree, so the result
// does not depend on scheduling.
template <typename T>
__global__ void __launch_bounds__(1024)
sce_loss_kernel(const T* __restrict__ logits, const void* __restrict__ targets, const float* __restrict__ row_stats,
                T* __restrict__ loss, int64_t rows, int64_t C, int32_t idx_dtype, unsigned long long* bad) {
  __shared__ float red[32];
  float acc = 0.0f;
  unsigned long long my_bad = 0;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    const int64_t t = load_index(targets, r, idx_dtype);
    float xt = 0.0f;
    if (t < 0 || t >= C) ++my_bad; else xt = ld_f32<T>(logits[r * C + t]);
    acc += logf(fmaxf(row_stats[2 * r + 1], 1.0e-7f)) - (xt - row_stats[2 * r]);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) loss[0] = st_f32<T>(rows > 0 ? v / static_cast<float>(rows) : 0.0f);
  }
  if (bad != nullptr && my_bad != 0) atomicAdd(bad, my_bad);
}

// grad[r, c] = (softmax[r, c] - (c == target[r])) * inv_n; one 16-byte vector per thread.
template <typename T, int VEC>
__global__ void sce_backward_kernel(const T* __restrict__ sm, const void* __restrict__ targets, T* __restrict__ grad,
                                    int64_t rows, int64_t C, int32_t idx_dtype, float inv_n) {
  using P = Pack<T, VEC>;
  const int64_t vec_per_row = C / VEC;
  const int64_t n = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int64_t c0 = (i - r * vec_per_row) * VEC;
    const int64_t t = load_index(targets, r, idx_dtype);
    P v = reinterpret_cast<const P*>(sm)[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float p = ld_f32<T>(v.e[e]);
      if (c0 + e == t) p += -1.0f;
      v.e[e] = st_f32<T>(p * inv_n);
    }
    reinterpret_cast<P*>(grad)[i] = v;
  }
}

__device__ __forceinline__ void atomic_add_elem(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_elem(__half* p, __half v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_elem(__nv_bfloat16* p, __nv_bfloat16 v) { atomicAdd(p, v); }

// inout[p, idx[i], q] += src[p, i, q]; one thread per src element, atomics because indices may repeat.
template <typename T>
__global__ void scatter_add_kernel(T* __restrict__ inout, const void* __restrict__ idx, const T* __restrict__ src,
                                   int64_t pre, int64_t axis_len, int64_t post, int64_t n_idx, int32_t idx_dtype,
                                   unsigned long long* bad) {
  const int64_t n = pre * n_idx * post;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < n;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t q = e % post;
    const int64_t pi = e / post;
    const int64_t i = pi % n_idx;
    const int64_t p = pi / n_idx;
    const int64_t t = load_index(idx, i, idx_dtype);
    if (t < 0 || t >= axis_len) {
      if (bad != nullptr && q == 0) atomicAdd(bad, 1ull);
      continue;
    }
    atomic_add_elem(inout + (p * axis_len + t) * post + q, src[e]);
  }
}

int grid_for(int64_t work_items, int threads, int sm_count) {
  const int64_t want = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count) * 16;
  return static_cast<int>(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace
}  // namespace nova

using namespace nova;

// ---------------------------------------------------------------- layer norm folded into a contraction
//
// Per row {mean, rstd} in fp32 from ONE read of x (the layer_norm reduction without its output pass): a warp
// per row, 16-byte loads, eight in flight per lane.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) row_stats_kernel(const T* __restrict__ x, float2* __restrict__ stats, int64_t rows, int32_t D) {
  using P = Pack<T, VEC>;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int nvec = D / VEC;
  for (int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const P* xr = reinterpret_cast<const P*>(x + row * D);
    float s0 = 0.0f, s1 = 0.0f;
    if constexpr (VEC > 1) {  // packed fp32 arithmetic; vectors past the row are zeros and add nothing
      const uint4* xv = reinterpret_cast<const uint4*>(xr);
      float2 a0 = make_float2(0.0f, 0.0f), a1 = make_float2(0.0f, 0.0f);
      for (int i0 = lane; i0 < nvec; i0 += 32 * 8) {
        uint4 pk[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) pk[u] = i0 + u * 32 < nvec ? xv[i0 + u * 32] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          for_pairs<T>(pk[u], [&](int, float2 v) {
            a0 = __fadd2_rn(a0, v);
            a1 = __ffma2_rn(v, v, a1);
          });
      }
      s0 = a0.x + a0.y;
      s1 = a1.x + a1.y;
    } else {
    for (int i0 = lane; i0 < nvec; i0 += 32 * 8) {
      P pk[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i0 + u * 32 < nvec) pk[u] = xr[i0 + u * 32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (i0 + u * 32 < nvec) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const float v = ld_f32<T>(pk[u].e[e]);
            s0 += v;
            s1 = fmaf(v, v, s1);
          }
        }
      }
    }
    }
    s0 = warp_sum(s0);
    s1 = warp_sum(s1);
    if (lane == 0) {
      const float inv_d = 1.0f / static_cast<float>(D);
      const float mean = s0 * inv_d;
      stats[row] = make_float2(mean, rsqrtf(s1 * inv_d - mean * mean + 1e-5f));
    }
  }
}

// W'[k, j] = round(gamma[k] * W[k, j]);  c[j] = sum_k W'[k, j];  d[j] = sum_k beta[k] * W[k, j] (+ bias[j]).
// One thread per column (coalesced along j), k ascending: a fixed summation order.  Runs once per weight.
template <typename T>
__global__ void ln_fold_prepare_kernel(const T* __restrict__ w, const T* __restrict__ gamma, const T* __restrict__ beta,
                                       const T* __restrict__ bias, T* __restrict__ wprime, float* __restrict__ cd, int64_t K,
                                       int64_t N, int64_t ldw) {
  const int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (j >= N) return;
  float c = 0.0f, d = bias ? ld_f32<T>(bias[j]) : 0.0f;
#pragma unroll 8
  for (int64_t k = 0; k < K; ++k) {
    const float wv = ld_f32<T>(w[k * ldw + j]);
    const T wp = st_f32<T>(ld_f32<T>(gamma[k]) * wv);
    wprime[k * N + j] = wp;
    c += ld_f32<T>(wp);
    d = fmaf(ld_f32<T>(beta[k]), wv, d);
  }
  cd[j] = c;
  cd[N + j] = d;
}

// ---------------------------------------------------------------- multi-GPU: re-interleave all-gathered column slabs
//
// After an all-gather every rank holds the ranks' output slabs one after the other, staging[r] = [rows, wmax] with
// the first width(r) columns valid.  This kernel writes the row-major [rows, cols] matrix: one thread per 16-byte
// chunk of the output (element-wise when a slab boundary or the row pitch is not 16-byte aligned), reads and writes
// both coalesced along rows.
struct SlabLayout {
  int32_t world;
  int64_t start[17];  // slab r covers columns [start[r], start[r + 1])
};

template <int kUnitBytes>
__global__ void interleave_slabs_kernel(const uint8_t* __restrict__ staging, uint8_t* __restrict__ out, int64_t rows,
                                        int64_t units_per_row, int64_t wmax_units, SlabLayout lay) {
  // everything is counted in units of kUnitBytes (16-byte chunks, or single elements)
  const int64_t n = rows * units_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / units_per_row;
    const int64_t c = i - row * units_per_row;
    int r = 0;
    while (r + 1 < lay.world && c >= lay.start[r + 1]) ++r;
    const uint8_t* src = staging + ((static_cast<int64_t>(r) * rows + row) * wmax_units + (c - lay.start[r])) * kUnitBytes;
    uint8_t* dst = out + i * kUnitBytes;
    if (kUnitBytes == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    else if (kUnitBytes == 4) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
    else *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src);
  }
}

namespace {
// The finish kernel is launched with programmatic stream serialization: it is scheduled while the main kernel's last
// CTAs still run and blocks in griddepcontrol.wait until that grid has ended, so its launch latency is off the
// critical path.  (Kernels that never call launch_dependents release their dependents when they end: the attribute
// is safe after any of the main kernels.)
template <typename T>
int32_t launch_finish_t(const float* partial, int n_partials, int64_t D, void* dgamma, void* dbeta, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((D + 31) / 32), 1, 1);
  cfg.blockDim = dim3(32, 32, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = options().pdl.load() != 0 ? 1 : 0;
  NOVA_CUDA_OK(cudaLaunchKernelEx(&cfg, ln_backward_finish_kernel<T>, partial, static_cast<int32_t>(n_partials),
                                  static_cast<int32_t>(D), static_cast<T*>(dgamma), static_cast<T*>(dbeta)));
  return NOVA_B200_OK;
}
int32_t launch_ln_backward_finish(const float* partial, int n_partials, int64_t D, int32_t dtype, void* dgamma, void* dbeta,
                                  cudaStream_t s) {
  if (dtype == NOVA_B200_F32) return launch_finish_t<float>(partial, n_partials, D, dgamma, dbeta, s);
  if (dtype == NOVA_B200_F16) return launch_finish_t<__half>(partial, n_partials, D, dgamma, dbeta, s);
  return launch_finish_t<__nv_bfloat16>(partial, n_partials, D, dgamma, dbeta, s);
}
}  // namespace

extern "C" {

int32_t nova_b200_layer_norm(const void* x, const void* gamma, const void* beta, void* y, void* mean_sum, void* rstd,
                             int64_t rows, int64_t D, int32_t dtype, void* stream) {
  if (rows < 0 || D < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "layer_norm: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "layer_norm: dtype must be f32, f16 or bf16");
  if (D > (1ll << 30)) return fail(NOVA_B200_ERR_TOO_LARGE, "layer_norm: D exceeds 2^30");
  if (rows == 0 || D == 0) return NOVA_B200_OK;
  if (!x || !gamma || !beta || !y) return fail(NOVA_B200_ERR_INVALID_ARG, "layer_norm: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_layer_norm: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, y, "nova_b200_layer_norm: the output")) != NOVA_B200_OK) return st;
  return dispatch_row_kernel<0>(x, gamma, beta, y, mean_sum, rstd, rows, D, dtype, ctx->sm_count,
                                static_cast<cudaStream_t>(stream), nullptr, ctx->status_word);
}

int32_t nova_b200_layer_norm_backward(const void* grad_y, const void* x, const void* gamma, const void* mean_sum,
                                      const void* rstd, void* dx, void* dgamma, void* dbeta, int64_t rows, int64_t D,
                                      int32_t dtype, void* stream) {
  if (rows < 0 || D < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "layer_norm_backward: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "layer_norm_backward: dtype must be f32, f16 or bf16");
  if (D == 0) return NOVA_B200_OK;
  if (!dgamma || !dbeta) return fail(NOVA_B200_ERR_INVALID_ARG, "layer_norm_backward: null pointer");
  if (rows > 0 && (!grad_y || !x || !gamma || !mean_sum || !rstd || !dx))
    return fail(NOVA_B200_ERR_INVALID_ARG, "layer_norm_backward: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_layer_norm_backward: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, dx, "nova_b200_layer_norm_backward: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype);
  const uintptr_t align = reinterpret_cast<uintptr_t>(grad_y) | reinterpret_cast<uintptr_t>(x) |
                          reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(dx);
  const int vec = (align % 16 == 0 && (D * es) % 16 == 0) ? 16 / es : 1;
  const int64_t nvec = D / vec;
  if (nvec > static_cast<int64_t>(kRowThreads) * 8)
    return fail(NOVA_B200_ERR_UNSUPPORTED,
                "layer_norm_backward: rows longer than 2048 sixteen-byte vectors (or 2048 elements when unaligned)");
  // One vector per thread (64 registers, 2048 resident threads per SM) for rows of up to 1024 vectors; longer rows
  // keep 2-8 vectors per thread in 256-thread CTAs.  Threads: a multiple of 32 covering the row.
  // rows of 2 KB .. 16 KB whose pointers allow bulk copies: the shared-memory ring kernel
  // (measured slower than the register kernels below on [8192, 4096] bf16, 2.3 against 3.0 TB/s, whatever the ring
  // depth or the CTAs per SM, so it is off unless asked for: option "ring_rows" = 2)
  if (vec > 1 && nvec >= 128 && nvec <= 1024 && options().ring_rows.load() == 2 &&
      reinterpret_cast<uintptr_t>(dx) % 16 == 0) {
    const size_t row_bytes = static_cast<size_t>(D) * es;
    int grid = 0;
    float* partial = nullptr;
    // two CTAs per SM share ~192 KB of ring: as many (grad_y, x) row slots per CTA as fit in 96 KB (2..8)
    int stages = static_cast<int>(std::max<size_t>(2, std::min<size_t>(kRingMaxStages, (96u << 10) / (2 * row_bytes))));
    if (const int64_t o = options().ring_stages.load(); o >= 2 && o <= kRingMaxStages) stages = static_cast<int>(o);
#define NOVA_LNB_RING(T, MAXV_)                                                                                       \
    do {                                                                                                              \
      auto kernel = ln_backward_ring_kernel<T, MAXV_, 512>;                                                           \
      const size_t smem = stages * 2 * row_bytes;                                                                     \
      int resident = ring_resident_ctas(kernel, 512, smem);                                                           \
      if (resident <= 0) return fail(NOVA_B200_ERR_CUDA, std::string("layer_norm_backward: the ring kernel cannot be configured: ") + nova_b200_last_error_string()); \
      if (const int64_t o = options().ring_ctas.load(); o >= 1 && o < resident) resident = static_cast<int>(o);       \
      grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(rows, static_cast<int64_t>(ctx->sm_count) * resident))); \
      void* scratch = nullptr;                                                                                        \
      st = acquire_scratch(ctx, s, static_cast<size_t>(grid) * 2 * D * sizeof(float), &scratch);                      \
      if (st != NOVA_B200_OK) return st;                                                                              \
      partial = static_cast<float*>(scratch);                                                                         \
      kernel<<<grid, 512, smem, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x), static_cast<const T*>(gamma), \
                                     static_cast<const T*>(mean_sum), static_cast<const T*>(rstd), static_cast<T*>(dx), partial, \
                                     rows, static_cast<int32_t>(D), stages, ctx->status_word);                        \
    } while (0)
#define NOVA_LNB_RING_T(T)                                            \
    do {                                                              \
      if (nvec <= 512) NOVA_LNB_RING(T, 1); else NOVA_LNB_RING(T, 2); \
    } while (0)
    if (dtype == NOVA_B200_F32) NOVA_LNB_RING_T(float);
    else if (dtype == NOVA_B200_F16) NOVA_LNB_RING_T(__half);
    else NOVA_LNB_RING_T(__nv_bfloat16);
#undef NOVA_LNB_RING_T
#undef NOVA_LNB_RING
    NOVA_CUDA_OK(cudaGetLastError());
    return launch_ln_backward_finish(partial, grid, D, dtype, dgamma, dbeta, s);
  }
  const bool wide = nvec <= 1024;
  const int threads = static_cast<int>(wide ? (nvec + 31) / 32 * 32 : kRowThreads);
  const int per_thread = static_cast<int>((nvec + threads - 1) / threads);
  const int max_v = per_thread <= 1 ? 1 : per_thread <= 2 ? 2 : per_thread <= 4 ? 4 : 8;
  // few persistent CTAs: every CTA ends with 2*D floats of column sums that the finish kernel has to read back.
  // Rows of up to 512 vectors, vectorised: the packed-arithmetic kernel, two rows per trip in 64 registers so that
  // 1024 threads are resident per SM (measured on [8192, 4096] bf16: 47.2 us; four rows per trip in one 128-register
  // CTA per SM, option "ring_ctas" = 1: 48.6 us; the scalar-arithmetic form, option "ring_rows" = 0: 67.8 us).
  const bool packed = wide && vec > 1 && threads <= 512 && options().ring_rows.load() != 0;
  const bool packed_wide = wide && vec > 1 && threads > 512 && options().ring_rows.load() != 0;  // one 1024-thread CTA per SM
  const bool two_ctas = packed && options().ring_ctas.load() != 1;
  const int rows_per = threads <= 512 ? (two_ctas ? 2 : 4) : 1;
  int resident = !wide ? (max_v >= 4 ? 1 : 2)
                       : packed_wide ? 1
                       : two_ctas ? std::max(2, std::min(16, 1024 / threads))
                                  : (rows_per == 4 ? std::max(1, std::min(4, 512 / threads)) : std::max(1, 2048 / threads));
  const int64_t row_blocks = wide ? (rows + rows_per - 1) / rows_per : rows;
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(row_blocks, static_cast<int64_t>(ctx->sm_count) * resident)));
  void* scratch = nullptr;
  st = acquire_scratch(ctx, s, static_cast<size_t>(grid) * 2 * D * sizeof(float), &scratch);
  if (st != NOVA_B200_OK) return st;
  float* partial = static_cast<float*>(scratch);
#define NOVA_LNB(T, V, MV)                                                                                             \
  ln_backward_kernel<T, V, MV, (MV) == 1 ? 1024 : kRowThreads><<<grid, threads, 0, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x),      \
                                                        static_cast<const T*>(gamma), static_cast<const T*>(mean_sum), \
                                                        static_cast<const T*>(rstd), static_cast<T*>(dx), partial,     \
                                                        rows, static_cast<int32_t>(D))
#define NOVA_LNB_ROWS(T, V, R, B)                                                                                     \
  ln_backward_rows_kernel<T, V, R, B><<<grid, threads, 0, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x), \
                                                              static_cast<const T*>(gamma), static_cast<const T*>(mean_sum), \
                                                              static_cast<const T*>(rstd), static_cast<T*>(dx), partial, rows, \
                                                              static_cast<int32_t>(D))
#define NOVA_LNB_PACKED(T)                                                                                            \
  ln_backward_packed_kernel<T, 4, 512, 1><<<grid, threads, 0, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x), \
                                                               static_cast<const T*>(gamma), static_cast<const T*>(mean_sum), \
                                                               static_cast<const T*>(rstd), static_cast<T*>(dx), partial, rows, \
                                                               static_cast<int32_t>(D))
#define NOVA_LNB_PACKED2(T)                                                                                           \
  ln_backward_packed_kernel<T, 2, 512, 2><<<grid, threads, 0, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x), \
                                                               static_cast<const T*>(gamma), static_cast<const T*>(mean_sum), \
                                                               static_cast<const T*>(rstd), static_cast<T*>(dx), partial, rows, \
                                                               static_cast<int32_t>(D))
#define NOVA_LNB_PACKED_WIDE(T)                                                                                       \
  ln_backward_packed_kernel<T, 1, 1024, 1><<<grid, threads, 0, s>>>(static_cast<const T*>(grad_y), static_cast<const T*>(x), \
                                                               static_cast<const T*>(gamma), static_cast<const T*>(mean_sum), \
                                                               static_cast<const T*>(rstd), static_cast<T*>(dx), partial, rows, \
                                                               static_cast<int32_t>(D))
#define NOVA_LNB_MV(T, V)                                                                       \
  do {                                                                                          \
    if (packed_wide && V > 1) NOVA_LNB_PACKED_WIDE(T);                                          \
    else if (two_ctas && V > 1) NOVA_LNB_PACKED2(T);                                            \
    else if (wide && rows_per == 4 && V > 1 && packed) NOVA_LNB_PACKED(T);                      \
    else if (wide && rows_per == 4) NOVA_LNB_ROWS(T, V, 4, 512);                                \
    else if (max_v == 1) NOVA_LNB(T, V, 1); else if (max_v == 2) NOVA_LNB(T, V, 2);             \
    else if (max_v == 4) NOVA_LNB(T, V, 4); else NOVA_LNB(T, V, 8);                             \
  } while (0)
  if (dtype == NOVA_B200_F32) { if (vec > 1) NOVA_LNB_MV(float, 4); else NOVA_LNB_MV(float, 1); }
  else if (dtype == NOVA_B200_F16) { if (vec > 1) NOVA_LNB_MV(__half, 8); else NOVA_LNB_MV(__half, 1); }
  else { if (vec > 1) NOVA_LNB_MV(__nv_bfloat16, 8); else NOVA_LNB_MV(__nv_bfloat16, 1); }
#undef NOVA_LNB_MV
#undef NOVA_LNB_PACKED
#undef NOVA_LNB_PACKED2
#undef NOVA_LNB_PACKED_WIDE
#undef NOVA_LNB_ROWS
#undef NOVA_LNB
  NOVA_CUDA_OK(cudaGetLastError());
  return launch_ln_backward_finish(partial, grid, D, dtype, dgamma, dbeta, s);
}

int32_t nova_b200_softmax(const void* x, void* y, int64_t rows, int64_t D, int32_t dtype, void* stream) {
  if (rows < 0 || D < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "softmax: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "softmax: dtype must be f32, f16 or bf16");
  if (D > (1ll << 30)) return fail(NOVA_B200_ERR_TOO_LARGE, "softmax: D exceeds 2^30");
  if (rows == 0 || D == 0) return NOVA_B200_OK;
  if (!x || !y) return fail(NOVA_B200_ERR_INVALID_ARG, "softmax: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_softmax: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, y, "nova_b200_softmax: the output")) != NOVA_B200_OK) return st;
  return dispatch_row_kernel<1>(x, nullptr, nullptr, y, nullptr, nullptr, rows, D, dtype, ctx->sm_count,
                                static_cast<cudaStream_t>(stream), nullptr, ctx->status_word);
}

static bool is_index_dtype(int32_t dt) { return dt == NOVA_B200_I16 || dt == NOVA_B200_I32 || dt == NOVA_B200_I64; }

int32_t nova_b200_sce(const void* logits, const void* targets, void* softmax_out, void* loss_out, int64_t rows, int64_t C,
                      int32_t dtype, int32_t idx_dtype, int64_t* bad_count, void* stream) {
  if (rows < 0 || C < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "sce: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "sce: dtype must be f32, f16 or bf16");
  if (!is_index_dtype(idx_dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "sce: target dtype must be i16, i32 or i64");
  if (C > (1ll << 30)) return fail(NOVA_B200_ERR_TOO_LARGE, "sce: C exceeds 2^30");
  if (!loss_out) return fail(NOVA_B200_ERR_INVALID_ARG, "sce: null pointer");
  if (rows > 0 && C > 0 && (!logits || !targets || !softmax_out)) return fail(NOVA_B200_ERR_INVALID_ARG, "sce: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, logits, "nova_b200_sce: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, softmax_out, "nova_b200_sce: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* scratch = nullptr;
  st = acquire_scratch(ctx, s, static_cast<size_t>(std::max<int64_t>(rows, 1)) * 2 * sizeof(float), &scratch);
  if (st != NOVA_B200_OK) return st;
  float* stats = static_cast<float*>(scratch);
  if (rows > 0 && C > 0) {
    st = dispatch_row_kernel<1>(logits, nullptr, nullptr, softmax_out, nullptr, nullptr, rows, C, dtype, ctx->sm_count, s, stats,
                                ctx->status_word);
    if (st != NOVA_B200_OK) return st;
  }
  const int64_t loss_rows = C > 0 ? rows : 0;
  auto* bad = reinterpret_cast<unsigned long long*>(bad_count);
  if (dtype == NOVA_B200_F32)
    sce_loss_kernel<float><<<1, 1024, 0, s>>>(static_cast<const float*>(logits), targets, stats, static_cast<float*>(loss_out), loss_rows, C, idx_dtype, bad);
  else if (dtype == NOVA_B200_F16)
    sce_loss_kernel<__half><<<1, 1024, 0, s>>>(static_cast<const __half*>(logits), targets, stats, static_cast<__half*>(loss_out), loss_rows, C, idx_dtype, bad);
  else
    sce_loss_kernel<__nv_bfloat16><<<1, 1024, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), targets, stats, static_cast<__nv_bfloat16*>(loss_out), loss_rows, C, idx_dtype, bad);
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_sce_backward(const void* softmax, const void* targets, void* grad, int64_t rows, int64_t C, int32_t dtype,
                               int32_t idx_dtype, void* stream) {
  return nova_b200_sce_backward_scaled(softmax, targets, grad, rows, C, dtype, idx_dtype, 1.0f, stream);
}

int32_t nova_b200_sce_backward_scaled(const void* softmax, const void* targets, void* grad, int64_t rows, int64_t C,
                                      int32_t dtype, int32_t idx_dtype, float scale, void* stream) {
  if (rows < 0 || C < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "sce_backward: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "sce_backward: dtype must be f32, f16 or bf16");
  if (!is_index_dtype(idx_dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "sce_backward: target dtype must be i16, i32 or i64");
  if (rows == 0 || C == 0) return NOVA_B200_OK;
  if (!softmax || !targets || !grad) return fail(NOVA_B200_ERR_INVALID_ARG, "sce_backward: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, softmax, "nova_b200_sce_backward: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, grad, "nova_b200_sce_backward: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype), vec = 16 / es;
  const bool vec_ok = C % vec == 0 && reinterpret_cast<uintptr_t>(softmax) % 16 == 0 && reinterpret_cast<uintptr_t>(grad) % 16 == 0;
  // one multiplier per element: (1 / rows) rounded to fp32 as the reference's constant is, times the caller's scale
  const float inv_n = static_cast<float>(1.0 / static_cast<double>(rows)) * scale;
  const int threads = 256;
  const int grid = grid_for(vec_ok ? rows * C / vec : rows * C, threads, ctx->sm_count);
#define NOVA_SCEB(T, V)                                                                                                  \
  sce_backward_kernel<T, V><<<grid, threads, 0, s>>>(static_cast<const T*>(softmax), targets, static_cast<T*>(grad), rows, C, \
                                                     idx_dtype, inv_n)
  if (dtype == NOVA_B200_F32) { if (vec_ok) NOVA_SCEB(float, 4); else NOVA_SCEB(float, 1); }
  else if (dtype == NOVA_B200_F16) { if (vec_ok) NOVA_SCEB(__half, 8); else NOVA_SCEB(__half, 1); }
  else { if (vec_ok) NOVA_SCEB(__nv_bfloat16, 8); else NOVA_SCEB(__nv_bfloat16, 1); }
#undef NOVA_SCEB
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_scatter_add(void* inout, const void* idx, const void* src, int64_t pre, int64_t axis_len, int64_t post,
                              int64_t n_idx, int32_t idx_dtype, int32_t dtype, int64_t* bad_count, void* stream) {
  if (pre < 0 || axis_len < 0 || post < 0 || n_idx < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "scatter_add: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "scatter_add: dtype must be f32, f16 or bf16");
  if (!is_index_dtype(idx_dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "scatter_add: index dtype must be i16, i32 or i64");
  if (pre == 0 || post == 0 || n_idx == 0) return NOVA_B200_OK;
  if (!inout || !idx || !src) return fail(NOVA_B200_ERR_INVALID_ARG, "scatter_add: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, src, "nova_b200_scatter_add: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, inout, "nova_b200_scatter_add: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const int grid = grid_for(pre * n_idx * post, threads, ctx->sm_count);
  auto* bad = reinterpret_cast<unsigned long long*>(bad_count);
  if (dtype == NOVA_B200_F32)
    scatter_add_kernel<float><<<grid, threads, 0, s>>>(static_cast<float*>(inout), idx, static_cast<const float*>(src), pre, axis_len, post, n_idx, idx_dtype, bad);
  else if (dtype == NOVA_B200_F16)
    scatter_add_kernel<__half><<<grid, threads, 0, s>>>(static_cast<__half*>(inout), idx, static_cast<const __half*>(src), pre, axis_len, post, n_idx, idx_dtype, bad);
  else
    scatter_add_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(static_cast<__nv_bfloat16*>(inout), idx, static_cast<const __nv_bfloat16*>(src), pre, axis_len, post, n_idx, idx_dtype, bad);
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_gather(const void* in, const void* idx, void* out, int64_t pre, int64_t axis_len, int64_t post,
                         int64_t n_idx, int32_t idx_dtype, int32_t batched_idx, int32_t elem_bytes,
                         int64_t* bad_count, void* stream) {
  if (pre < 0 || axis_len < 0 || post < 0 || n_idx < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "gather: negative extent");
  if (idx_dtype != NOVA_B200_I16 && idx_dtype != NOVA_B200_I32 && idx_dtype != NOVA_B200_I64)
    return fail(NOVA_B200_ERR_UNSUPPORTED, "gather: index dtype must be i16, i32 or i64");
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
    return fail(NOVA_B200_ERR_UNSUPPORTED, "gather: element size must be 1, 2, 4 or 8 bytes");
  if (pre == 0 || post == 0 || n_idx == 0) return NOVA_B200_OK;
  if (!in || !idx || !out) return fail(NOVA_B200_ERR_INVALID_ARG, "gather: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, in, "nova_b200_gather: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, out, "nova_b200_gather: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t row_bytes = post * elem_bytes;
  const uintptr_t align = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                          static_cast<uintptr_t>(row_bytes);
  auto* bad = reinterpret_cast<unsigned long long*>(bad_count);
  const int threads = 256;
#define NOVA_GATHER(U)                                                                                          \
  do {                                                                                                          \
    const int64_t units = row_bytes / static_cast<int64_t>(sizeof(U));                                          \
    int g_shift = 0;                                                                                            \
    while (g_shift < 5 && (int64_t(1) << g_shift) < units) ++g_shift;                                           \
    gather_kernel<U><<<grid_for((pre * n_idx) << g_shift, threads, ctx->sm_count), threads, 0, s>>>(            \
        static_cast<const U*>(in), idx, static_cast<U*>(out), pre, axis_len, units, n_idx, idx_dtype,           \
        batched_idx, g_shift, bad);                                                                             \
  } while (0)
  if (align % 16 == 0) NOVA_GATHER(uint4);
  else if (align % 8 == 0) NOVA_GATHER(uint2);
  else if (align % 4 == 0) NOVA_GATHER(uint32_t);
  else if (align % 2 == 0) NOVA_GATHER(uint16_t);
  else NOVA_GATHER(uint8_t);
#undef NOVA_GATHER
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_column_sum(const void* x, void* out, int64_t rows, int64_t cols, int32_t dtype, void* stream) {
  if (rows < 0 || cols < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "column_sum: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "column_sum: dtype must be f32, f16 or bf16");
  if (cols == 0) return NOVA_B200_OK;
  if (!out || (rows > 0 && !x)) return fail(NOVA_B200_ERR_INVALID_ARG, "column_sum: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_column_sum: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, out, "nova_b200_column_sum: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t col_tiles = (cols + 63) / 64;
  // enough row splits to fill the machine, at most one per 8 rows
  int64_t splits = (static_cast<int64_t>(ctx->sm_count) * 8 + col_tiles - 1) / col_tiles;
  splits = std::max<int64_t>(1, std::min<int64_t>(splits, (rows + 7) / 8));
  splits = std::min<int64_t>(splits, 65535);
  void* scratch = nullptr;  // the partial sums live in this stream's scratch
  st = acquire_scratch(ctx, s, static_cast<size_t>(splits * cols) * sizeof(float), &scratch);
  if (st != NOVA_B200_OK) return st;
  float* partial = static_cast<float*>(scratch);
  const dim3 grid(static_cast<unsigned>(col_tiles), static_cast<unsigned>(splits));
  const int fgrid = grid_for(cols, 256, ctx->sm_count);
#define NOVA_COLSUM(T)                                                                                   \
  do {                                                                                                   \
    column_sum_partial_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), partial, rows, cols);    \
    column_sum_final_kernel<T><<<fgrid, 256, 0, s>>>(partial, static_cast<T*>(out), cols, static_cast<int>(splits)); \
  } while (0)
  if (dtype == NOVA_B200_F32) NOVA_COLSUM(float);
  else if (dtype == NOVA_B200_F16) NOVA_COLSUM(__half);
  else NOVA_COLSUM(__nv_bfloat16);
#undef NOVA_COLSUM
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_activation(const void* x, void* y, int64_t n, int32_t dtype, int32_t act, void* stream) {
  if (n < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "activation: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "activation: dtype must be f32, f16 or bf16");
  if (act < NOVA_B200_ACT_NONE || act > NOVA_B200_ACT_GELU_TANH)
    return fail(NOVA_B200_ERR_INVALID_ARG, "activation: unknown activation");
  if (n == 0) return NOVA_B200_OK;
  if (!x || !y) return fail(NOVA_B200_ERR_INVALID_ARG, "activation: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_activation: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, y, "nova_b200_activation: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype), vec = 16 / es;
  const bool vec_ok = n % vec == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
  const int threads = 256;
  const int grid = grid_for(vec_ok ? n / vec : n, threads, ctx->sm_count);
#define NOVA_ACT(T, V) activation_kernel<T, V><<<grid, threads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), n, act)
  if (dtype == NOVA_B200_F32) { if (vec_ok) NOVA_ACT(float, 4); else NOVA_ACT(float, 1); }
  else if (dtype == NOVA_B200_F16) { if (vec_ok) NOVA_ACT(__half, 8); else NOVA_ACT(__half, 1); }
  else { if (vec_ok) NOVA_ACT(__nv_bfloat16, 8); else NOVA_ACT(__nv_bfloat16, 1); }
#undef NOVA_ACT
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_gelu_backward(const void* go, const void* x, void* y, int64_t n, int32_t dtype, void* stream) {
  if (n < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "gelu_backward: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "gelu_backward: dtype must be f32, f16 or bf16");
  if (n == 0) return NOVA_B200_OK;
  if (!go || !x || !y) return fail(NOVA_B200_ERR_INVALID_ARG, "gelu_backward: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "nova_b200_gelu_backward: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, y, "nova_b200_gelu_backward: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype), vec = 16 / es;
  const bool vec_ok = n % vec == 0 && reinterpret_cast<uintptr_t>(go) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(y) % 16 == 0;
  const int threads = 256;
  const int grid = grid_for(vec_ok ? n / vec : n, threads, ctx->sm_count);
#define NOVA_GB(T, V) \
  gelu_backward_kernel<T, V><<<grid, threads, 0, s>>>(static_cast<const T*>(go), static_cast<const T*>(x), static_cast<T*>(y), n)
  if (dtype == NOVA_B200_F32) { if (vec_ok) NOVA_GB(float, 4); else NOVA_GB(float, 1); }
  else if (dtype == NOVA_B200_F16) { if (vec_ok) NOVA_GB(__half, 8); else NOVA_GB(__half, 1); }
  else { if (vec_ok) NOVA_GB(__nv_bfloat16, 8); else NOVA_GB(__nv_bfloat16, 1); }
#undef NOVA_GB
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_add_rowbcast(const void* a, const void* b, void* out, int64_t rows, int64_t cols, int32_t b_is_full,
                               int32_t dtype, void* stream) {
  if (rows < 0 || cols < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "add: negative extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "add: dtype must be f32, f16 or bf16");
  if (rows == 0 || cols == 0) return NOVA_B200_OK;
  if (!a || !b || !out) return fail(NOVA_B200_ERR_INVALID_ARG, "add: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, a, "nova_b200_add_rowbcast: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, out, "nova_b200_add_rowbcast: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype), vec = 16 / es;
  const bool vec_ok = cols % vec == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(b) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const int threads = 256;
  const int grid = grid_for(vec_ok ? rows * cols / vec : rows * cols, threads, ctx->sm_count);
#define NOVA_ADD(T, V)                                                                                       \
  add_rowbcast_kernel<T, V><<<grid, threads, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b),      \
                                                     static_cast<T*>(out), rows, cols, b_is_full)
  if (dtype == NOVA_B200_F32) { if (vec_ok) NOVA_ADD(float, 4); else NOVA_ADD(float, 1); }
  else if (dtype == NOVA_B200_F16) { if (vec_ok) NOVA_ADD(__half, 8); else NOVA_ADD(__half, 1); }
  else { if (vec_ok) NOVA_ADD(__nv_bfloat16, 8); else NOVA_ADD(__nv_bfloat16, 1); }
#undef NOVA_ADD
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_binary(const void* a, const void* b, void* out, int32_t rank, const int64_t* shape,
                         const int64_t* a_strides, const int64_t* b_strides, int32_t op, int32_t dtype, void* stream) {
  if (rank < 0 || rank > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, "binary: rank must be 0..6");
  if (op < NOVA_B200_BIN_ADD || op > NOVA_B200_BIN_MUL) return fail(NOVA_B200_ERR_INVALID_ARG, "binary: unknown op");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "binary: dtype must be f32, f16 or bf16");
  if (rank > 0 && (!shape || !a_strides || !b_strides)) return fail(NOVA_B200_ERR_INVALID_ARG, "binary: null shape or strides");
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) {
    if (shape[i] < 0 || a_strides[i] < 0 || b_strides[i] < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "binary: negative extent or stride");
    n *= shape[i];
  }
  if (n == 0) return NOVA_B200_OK;
  if (!a || !b || !out) return fail(NOVA_B200_ERR_INVALID_ARG, "binary: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, a, "binary: an input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, out, "binary: the output")) != NOVA_B200_OK) return st;
  // drop size-1 dims, then merge neighbours that both operands walk like one dim
  BinaryDims d{};
  for (int i = 0; i < rank; ++i) {
    if (shape[i] == 1) continue;
    const int64_t sa = a_strides[i], sb = b_strides[i];
    if (d.rank > 0) {
      const int k = d.rank - 1;
      if (d.sa[k] == sa * shape[i] && d.sb[k] == sb * shape[i]) {  // (0 == 0 * n merges two broadcast dims too)
        d.shape[k] *= shape[i]; d.sa[k] = sa; d.sb[k] = sb;
        continue;
      }
    }
    d.shape[d.rank] = shape[i]; d.sa[d.rank] = sa; d.sb[d.rank] = sb;
    ++d.rank;
  }
  if (d.rank == 0) { d.rank = 1; d.shape[0] = 1; d.sa[0] = d.sb[0] = 0; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256, ctx->sm_count);
#define NOVA_BIN(T)                                                                                                      \
  do {                                                                                                                   \
    if (op == NOVA_B200_BIN_ADD) binary_broadcast_kernel<T, 0><<<grid, 256, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, d); \
    else if (op == NOVA_B200_BIN_SUB) binary_broadcast_kernel<T, 1><<<grid, 256, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, d); \
    else binary_broadcast_kernel<T, 2><<<grid, 256, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, d); \
  } while (0)
  if (dtype == NOVA_B200_F32) NOVA_BIN(float);
  else if (dtype == NOVA_B200_F16) NOVA_BIN(__half);
  else NOVA_BIN(__nv_bfloat16);
#undef NOVA_BIN
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_row_stats(const void* x, float* stats, int64_t rows, int64_t D, int32_t dtype, void* stream) {
  if (rows < 0 || D < 1) return fail(NOVA_B200_ERR_INVALID_ARG, "row_stats: bad extent");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "row_stats: dtype must be f32, f16 or bf16");
  if (D > (1ll << 30)) return fail(NOVA_B200_ERR_TOO_LARGE, "row_stats: D exceeds 2^30");
  if (rows == 0) return NOVA_B200_OK;
  if (!x || !stats) return fail(NOVA_B200_ERR_INVALID_ARG, "row_stats: null pointer");
  if (reinterpret_cast<uintptr_t>(stats) % 8 != 0) return fail(NOVA_B200_ERR_LAYOUT, "row_stats: stats must be 8-byte aligned");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, x, "row_stats: the input")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, stats, "row_stats: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int es = dtype_bytes(dtype), vec = 16 / es;
  const bool vec_ok = D % vec == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((rows + 7) / 8, static_cast<int64_t>(ctx->sm_count) * 8)));
  float2* out = reinterpret_cast<float2*>(stats);
  const int32_t d = static_cast<int32_t>(D);
  if (dtype == NOVA_B200_F32) { if (vec_ok) row_stats_kernel<float, 4><<<grid, 256, 0, s>>>(static_cast<const float*>(x), out, rows, d); else row_stats_kernel<float, 1><<<grid, 256, 0, s>>>(static_cast<const float*>(x), out, rows, d); }
  else if (dtype == NOVA_B200_F16) { if (vec_ok) row_stats_kernel<__half, 8><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), out, rows, d); else row_stats_kernel<__half, 1><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), out, rows, d); }
  else { if (vec_ok) row_stats_kernel<__nv_bfloat16, 8><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), out, rows, d); else row_stats_kernel<__nv_bfloat16, 1><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), out, rows, d); }
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_ln_fold_prepare(const void* w, const void* gamma, const void* beta, const void* bias, void* wprime, float* cd,
                                  int64_t K, int64_t N, int64_t ldw, int32_t dtype, void* stream) {
  if (K < 1 || N < 1 || ldw < N) return fail(NOVA_B200_ERR_INVALID_ARG, "ln_fold_prepare: bad extent or pitch");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "ln_fold_prepare: dtype must be f32, f16 or bf16");
  if (!w || !gamma || !beta || !wprime || !cd) return fail(NOVA_B200_ERR_INVALID_ARG, "ln_fold_prepare: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, w, "ln_fold_prepare: the weight")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, wprime, "ln_fold_prepare: the output")) != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>((N + 127) / 128);
#define NOVA_PREP(T)                                                                                                  \
  ln_fold_prepare_kernel<T><<<grid, 128, 0, s>>>(static_cast<const T*>(w), static_cast<const T*>(gamma), static_cast<const T*>(beta), \
                                                 static_cast<const T*>(bias), static_cast<T*>(wprime), cd, K, N, ldw)
  if (dtype == NOVA_B200_F32) NOVA_PREP(float);
  else if (dtype == NOVA_B200_F16) NOVA_PREP(__half);
  else NOVA_PREP(__nv_bfloat16);
#undef NOVA_PREP
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t nova_b200_interleave_slabs(const void* staging, void* out, int64_t rows, int64_t cols, int32_t world,
                                   int64_t slab_pitch, int64_t align, int32_t elem_bytes, void* stream) {
  if (rows < 0 || cols < 0 || world < 1 || world > 16 || align < 1 || slab_pitch < 0)
    return fail(NOVA_B200_ERR_INVALID_ARG, "interleave_slabs: bad extent (1 <= world <= 16)");
  if (elem_bytes != 2 && elem_bytes != 4) return fail(NOVA_B200_ERR_UNSUPPORTED, "interleave_slabs: 2- or 4-byte elements");
  if (rows == 0 || cols == 0) return NOVA_B200_OK;
  if (!staging || !out) return fail(NOVA_B200_ERR_INVALID_ARG, "interleave_slabs: null pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if ((st = check_pointer_device(ctx, staging, "interleave_slabs: the staging buffer")) != NOVA_B200_OK) return st;
  if ((st = check_pointer_device(ctx, out, "interleave_slabs: the output")) != NOVA_B200_OK) return st;
  // the partition of nova_compiler_b200/sharding.py column_slab: whole `align`-column units dealt out contiguously,
  // the first (units % world) ranks one unit more, the last non-empty slab takes the ragged remainder
  SlabLayout lay{};
  lay.world = world;
  const int64_t units = (cols + align - 1) / align, base = units / world, extra = units % world;
  int64_t widest = 0;
  for (int r = 0; r <= world; ++r) {
    const int64_t u = r * base + std::min<int64_t>(r, extra);
    lay.start[r] = std::min<int64_t>(u * align, cols);
    if (r > 0) widest = std::max(widest, lay.start[r] - lay.start[r - 1]);
  }
  if (slab_pitch < widest) return fail(NOVA_B200_ERR_LAYOUT, "interleave_slabs: slab_pitch is narrower than the widest slab");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per = 16 / elem_bytes;
  bool vec = (reinterpret_cast<uintptr_t>(staging) | reinterpret_cast<uintptr_t>(out)) % 16 == 0 && cols % per == 0 &&
             slab_pitch % per == 0;
  for (int r = 0; r <= world && vec; ++r) vec = lay.start[r] % per == 0;
  if (vec) {
    for (int r = 0; r <= world; ++r) lay.start[r] /= per;
    const int64_t n = rows * (cols / per);
    interleave_slabs_kernel<16><<<grid_for(n, 256, ctx->sm_count), 256, 0, s>>>(
        static_cast<const uint8_t*>(staging), static_cast<uint8_t*>(out), rows, cols / per, slab_pitch / per, lay);
  } else if (elem_bytes == 4) {
    interleave_slabs_kernel<4><<<grid_for(rows * cols, 256, ctx->sm_count), 256, 0, s>>>(
        static_cast<const uint8_t*>(staging), static_cast<uint8_t*>(out), rows, cols, slab_pitch, lay);
  } else {
    interleave_slabs_kernel<2><<<grid_for(rows * cols, 256, ctx->sm_count), 256, 0, s>>>(
        static_cast<const uint8_t*>(staging), static_cast<uint8_t*>(out), rows, cols, slab_pitch, lay);
  }
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

}  // extern "C"
