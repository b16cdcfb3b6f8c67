// HBM-bound kernels of the Flux DiT block path: LayerNorm + adaLN modulation, RMSNorm
// (forward and backward), RoPE, fused q/k/v assembly (split + QK-RMSNorm + RoPE + head-major
// concat), modulation scale/shift and gate/residual, SiLU, and the small-batch modulation
// projection (a GEMV over bf16 weights).
//
// Common shape of every kernel: 16-byte vector loads/stores, a row (or row segment) held in
// registers or, for rows of 2-24 KB, staged in shared memory by a bulk copy; fp32 statistics
// (one pass over staged rows, mean then centred variance over register-held rows), reductions
// by warp shuffles only.  Algorithmic traffic is "every input once, every output once"; nothing
// is staged through global scratch.  The 57-113 MB problems of the block are short enough
// (10-20 us) that issue slots, shared-memory traffic and the order in which requests are made
// decide their speed as much as the byte count does; the comments at each kernel say what was
// measured.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace fluxb {

// ----------------------------------------------------------------------------------------
// 16-byte vector access for fp32 / bf16 rows, presented to the math as fp32 lanes.
// ----------------------------------------------------------------------------------------
template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  float v[4];
  __device__ __forceinline__ void unpack(const uint4& t) {
    v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y);
    v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
  }
  __device__ __forceinline__ void load(const float* p) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ void load_nc(const float* p) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  float v[8];
  __device__ __forceinline__ void unpack(const uint4& t) {
    v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
    v[4] = bf16_lo(t.z); v[5] = bf16_hi(t.z); v[6] = bf16_lo(t.w); v[7] = bf16_hi(t.w);
  }
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    unpack(*reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ void load_nc(const __nv_bfloat16* p) {
    unpack(__ldg(reinterpret_cast<const uint4*>(p)));
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint4 t;
    t.x = pack_bf16(v[0], v[1]); t.y = pack_bf16(v[2], v[3]);
    t.z = pack_bf16(v[4], v[5]); t.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = t;
  }
};

// Makes the compiler forget what it knows about a packed vector, so the fp32 widening is redone
// at each use instead of being kept live (which doubles the registers of a bf16 row).
__device__ __forceinline__ void forget(uint4& t) {
  asm volatile("" : "+r"(t.x), "+r"(t.y), "+r"(t.z), "+r"(t.w));
}

__device__ __forceinline__ uint4 ld_nc_u4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Row addressing through a 3-level stride (head-split views): row -> element offset.
struct RowAddr {
  int64_t n1, n2, s0, s1, s2;
  // Set by the host when all rows follow each other at stride s2 (a contiguous tensor): no index
  // split then; the 64-bit divisions of the general case cost more than a 128-wide row's math.
  int flat;
  __device__ __forceinline__ int64_t offset(int64_t row) const {
    if (flat) return row * s2;
    if (row < (1ll << 31) && n1 < (1ll << 31) && n2 < (1ll << 31)) {
      const uint32_t r = (uint32_t)row, d2 = (uint32_t)n2, d1 = (uint32_t)n1;
      const uint32_t t = r / d2, i2 = r - t * d2, i0 = t / d1, i1 = t - i0 * d1;
      return (int64_t)i0 * s0 + (int64_t)i1 * s1 + (int64_t)i2 * s2;
    }
    const int64_t i2 = row % n2;
    const int64_t t = row / n2;
    return (t / n1) * s0 + (t % n1) * s1 + i2 * s2;
  }
};

// ----------------------------------------------------------------------------------------
// LayerNorm (no affine) + modulation.  G lanes own one row; each lane holds VPL vectors.
// cols == G * VPL * Vec<T>::N.
// ----------------------------------------------------------------------------------------
template <typename T, int G, int VPL>
__global__ void __launch_bounds__(256, (VPL <= 12 ? 3 : (VPL <= 24 ? 2 : 1)))
ln_mod_rows_kernel(const T* __restrict__ x, const T* __restrict__ scale, const T* __restrict__ shift,
                   T* __restrict__ y, int64_t rows, int cols, int64_t rows_per_batch, int64_t x_ld,
                   int64_t y_ld, int64_t mod_stride, float eps) {
  constexpr int VN = Vec<T>::N;
  const int lane_in_group = threadIdx.x % G;
  const int64_t groups_per_block = blockDim.x / G;
  const int64_t row = blockIdx.x * groups_per_block + threadIdx.x / G;
  const bool active = row < rows;
  const int64_t r = active ? row : rows - 1;  // keep every lane in the shuffles

  // The row stays packed (16 bytes per register quad) so that a 3072-wide bf16 row costs 48
  // registers per lane, not 96; values are widened to fp32 where they are used.
  uint4 raw[VPL];
  const T* xr = x + r * x_ld;
#pragma unroll
  for (int i = 0; i < VPL; ++i)
    raw[i] = *reinterpret_cast<const uint4*>(xr + (i * G + lane_in_group) * VN);

  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    Vec<T> t;
    t.unpack(raw[i]);
#pragma unroll
    for (int j = 0; j < VN; ++j) s += t.v[j];
  }
  const float mean = group_sum<G>(s) / cols;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    Vec<T> t;
    forget(raw[i]);
    t.unpack(raw[i]);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      float d = t.v[j] - mean;
      q += d * d;
    }
  }
  const float rstd = rsqrtf(group_sum<G>(q) / cols + eps);

  const int64_t b = r / rows_per_batch;
  const T* sc = scale + b * mod_stride;
  const T* sh = shift + b * mod_stride;
  T* yr = y + r * y_ld;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * G + lane_in_group) * VN;
    Vec<T> t, a, d;
    forget(raw[i]);
    t.unpack(raw[i]);
    a.load_nc(sc + c);
    d.load_nc(sh + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) t.v[j] = (t.v[j] - mean) * rstd * (1.0f + a.v[j]) + d.v[j];
    if (active) t.store(yr + c);
  }
}

// Any cols (multiple of the vector width): one warp per row, three passes over the row.
template <typename T>
__global__ void __launch_bounds__(256)
ln_mod_generic_kernel(const T* __restrict__ x, const T* __restrict__ scale,
                      const T* __restrict__ shift, T* __restrict__ y, int64_t rows, int cols,
                      int64_t rows_per_batch, int64_t x_ld, int64_t y_ld, int64_t mod_stride,
                      float eps) {
  constexpr int VN = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const T* xr = x + row * x_ld;
  float s = 0.f;
  for (int c = lane * VN; c < cols; c += 32 * VN) {
    Vec<T> t;
    t.load(xr + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) s += t.v[j];
  }
  const float mean = warp_sum(s) / cols;
  float q = 0.f;
  for (int c = lane * VN; c < cols; c += 32 * VN) {
    Vec<T> t;
    t.load(xr + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      float d = t.v[j] - mean;
      q += d * d;
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / cols + eps);
  const int64_t b = row / rows_per_batch;
  const T* sc = scale + b * mod_stride;
  const T* sh = shift + b * mod_stride;
  T* yr = y + row * y_ld;
  for (int c = lane * VN; c < cols; c += 32 * VN) {
    Vec<T> t, a, d;
    t.load(xr + c);
    a.load_nc(sc + c);
    d.load_nc(sh + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) t.v[j] = (t.v[j] - mean) * rstd * (1.0f + a.v[j]) + d.v[j];
    t.store(yr + c);
  }
}

// ----------------------------------------------------------------------------------------
// Wide rows (2 KB - 24 KB): the row is fetched by ONE bulk asynchronous copy into shared memory,
// one warp per row.  A row in flight costs no registers, so every row of a [4608, 3072] problem
// is resident at once (2 blocks of 16 rows per SM = one wave): all loads are issued in the first
// microsecond and rows are written back as they complete.
//
// Once a row has landed the warp's cost is shared-memory traffic (32 rows per SM land within a
// few microseconds of each other and share one 128 B/clock pipe), so the kernel touches the row
// as few times as it can: ONE pass for the statistics, one pass that reads the row again, applies
// the modulation and writes the result over it, and a bulk copy out.  With kStagedMod the
// per-column vectors (scale and shift, or the RMSNorm weight) are fetched once per block into
// shared memory instead of once per row through L1 (12 KB per 6 KB row otherwise).
//
// The LayerNorm statistics are the shifted one-pass form: with p = the row's first element,
// mean = p + E[x - p] and var = E[(x - p)^2] - E[x - p]^2, accumulated in fp32.  Shifting by an
// element of the row keeps the subtraction benign when |mean| >> std (the plain
// E[x^2] - mean^2 form is not).
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Waits (bounded) for a staged copy.  If the copy never lands the row stays unwritten, so the
// give-up is recorded in the device status word like every other bounded wait (site 71).
__device__ __forceinline__ bool wait_row(uint64_t* bar, DeviceStatus* status) {
  for (uint32_t spin = 0; spin < (1u << 24); ++spin)
    if (mbar_try_wait(bar, 0)) return true;
  report_error(status, FLUXB_ERR_TIMEOUT, 71);
  return false;
}

constexpr int kBulkHeaderBytes = 256;  // mbarriers: one per warp (up to 16) + one for the vectors

template <typename T, bool kLayerNorm, bool kStagedMod, int kVPL>
__global__ void __launch_bounds__(512, 2)
norm_rows_bulk_kernel(const T* __restrict__ x, const T* __restrict__ scale, const T* __restrict__ shift,
                      T* __restrict__ y, float* __restrict__ rstd_out, int64_t rows, int cols,
                      int64_t rows_per_batch, RowAddr xaddr, int64_t y_ld, int64_t mod_stride, float eps,
                      DeviceStatus* status) {
  constexpr int VN = Vec<T>::N;
  constexpr int kModVecs = kLayerNorm ? 2 : 1;
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem);  // [warps + 1]
  T* smod = reinterpret_cast<T*>(bulk_smem + kBulkHeaderBytes);
  T* srow = reinterpret_cast<T*>(bulk_smem + kBulkHeaderBytes + (kStagedMod ? kModVecs * (size_t)row_bytes : 0) +
                                 (size_t)warp * row_bytes);
  const int64_t row = (int64_t)blockIdx.x * warps + warp;
  // All rows of a block belong to one batch element when kStagedMod (the launcher checks).
  const int64_t batch = kLayerNorm ? ((int64_t)blockIdx.x * warps) / rows_per_batch : 0;
  // The per-column vectors are requested BEFORE any row of the block: requests are served roughly
  // in order, and a vector request queued behind thousands of row requests would land last and
  // hold every row's second pass until then.
  if (lane == 0) {
    mbar_init(&bars[warp], 1);
    if (kStagedMod && warp == 0) mbar_init(&bars[warps], 1);
    mbar_fence_init();
    fence_proxy_async_smem();
    if (kStagedMod && warp == 0) {
      mbar_expect_tx(&bars[warps], kModVecs * row_bytes);
      bulk_load_row(smod, scale + batch * mod_stride, row_bytes, &bars[warps]);
      if (kLayerNorm) bulk_load_row(smod + cols, shift + batch * mod_stride, row_bytes, &bars[warps]);
    }
  }
  if (kStagedMod) __syncthreads();  // the vectors' barrier is initialised before anyone polls it
  if (lane == 0 && row < rows) {
    mbar_expect_tx(&bars[warp], row_bytes);
    bulk_load_row(srow, x + xaddr.offset(row), row_bytes, &bars[warp]);
  }
  __syncwarp();
  if (row >= rows) return;  // whole warp leaves together; the warps do not meet again
  if (!wait_row(&bars[warp], status)) return;

  // kVPL > 0: the row is exactly kVPL vectors per lane and the loops unroll completely.
  const int nvec = kVPL > 0 ? kVPL * 32 : cols / VN;
  float mean = 0.f, rstd;
  if (kLayerNorm) {
    // 16-bit rows need no shift: their own quantisation (2^-9 of |x|) is 64 times the fp32
    // cancellation error of the unshifted form at any mean/std ratio.
    float pivot = 0.f;
    if (sizeof(T) > 2) {
      Vec<T> first;
      first.load(srow);
      pivot = first.v[0];
    }
    float s = 0.f, q = 0.f;
#pragma unroll(kVPL > 0 ? kVPL : 1)
    for (int i = lane; i < nvec; i += 32) {
      Vec<T> t;
      t.load(srow + i * VN);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        const float d = sizeof(T) > 2 ? t.v[j] - pivot : t.v[j];
        s += d;
        q = fmaf(d, d, q);
      }
    }
    const float ds = warp_sum(s) / cols;
    mean = pivot + ds;
    rstd = rsqrtf(fmaxf(warp_sum(q) / cols - ds * ds, 0.f) + eps);
  } else {
    float q = 0.f;
#pragma unroll(kVPL > 0 ? kVPL : 1)
    for (int i = lane; i < nvec; i += 32) {
      Vec<T> t;
      t.load(srow + i * VN);
#pragma unroll
      for (int j = 0; j < VN; ++j) q = fmaf(t.v[j], t.v[j], q);
    }
    rstd = rsqrtf(warp_sum(q) / cols + eps);
    if (rstd_out != nullptr && lane == 0) rstd_out[row] = rstd;
  }
  // The result replaces the row in shared memory and leaves as ONE bulk copy, like it came: the
  // lanes issue no global stores and the warp's last act is to wait until the copy engine has
  // read the staged row.
  T* yr = y + row * y_ld;
  if (kStagedMod) {
    if (!wait_row(&bars[warps], status)) return;
  }
  if (kLayerNorm) {
    const int64_t b = kStagedMod ? 0 : row / rows_per_batch;
    const T* sc = kStagedMod ? smod : scale + b * mod_stride;
    const T* sh = kStagedMod ? smod + cols : shift + b * mod_stride;
    const float neg_mean_rstd = -mean * rstd;  // (x - mean) * rstd as one fused multiply-add
#pragma unroll(kVPL > 0 ? kVPL : 1)
    for (int i = lane; i < nvec; i += 32) {
      Vec<T> t, a, d;
      t.load(srow + i * VN);
      if (kStagedMod) {
        a.load(sc + i * VN);
        d.load(sh + i * VN);
      } else {
        a.load_nc(sc + i * VN);
        d.load_nc(sh + i * VN);
      }
#pragma unroll
      for (int j = 0; j < VN; ++j) t.v[j] = fmaf(fmaf(t.v[j], rstd, neg_mean_rstd), 1.0f + a.v[j], d.v[j]);
      t.store(srow + i * VN);
    }
  } else {
#pragma unroll(kVPL > 0 ? kVPL : 1)
    for (int i = lane; i < nvec; i += 32) {
      Vec<T> t, wv;
      t.load(srow + i * VN);
      if (kStagedMod) wv.load(smod + i * VN);
      else wv.load_nc(scale + i * VN);
#pragma unroll
      for (int j = 0; j < VN; ++j) t.v[j] = t.v[j] * rstd * wv.v[j];
      t.store(srow + i * VN);
    }
  }
  fence_proxy_async_smem();  // each lane's writes, before the async proxy reads them
  __syncwarp();
  if (lane == 0) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(yr)),
                 "r"(smem_u32(srow)), "r"(row_bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  __syncwarp();
}

// True when the bulk-copy kernel applies: rows of 2-24 KB, 16-byte multiples, 16-byte aligned.
static inline bool bulk_rows_ok(int64_t cols, size_t elt, const RowAddr& a) {
  const int64_t row_bytes = cols * (int64_t)elt;
  if (row_bytes < 2048 || row_bytes > 24576 || row_bytes % 16) return false;
  return (a.s0 * (int64_t)elt) % 16 == 0 && (a.s1 * (int64_t)elt) % 16 == 0 && (a.s2 * (int64_t)elt) % 16 == 0;
}

template <typename T, bool kLayerNorm, bool kStagedMod>
static int launch_norm_bulk_as(const T* x, const T* scale, const T* shift, T* y, float* rstd, int64_t rows,
                               int64_t cols, int64_t rpb, RowAddr xaddr, int64_t y_ld, int64_t mod_stride,
                               float eps, cudaStream_t st) {
  const int warps = kStagedMod ? 16 : 8;
  const size_t smem = kBulkHeaderBytes + ((kStagedMod ? (kLayerNorm ? 2 : 1) : 0) + warps) * (size_t)cols * sizeof(T);
  // Rows of 12 vectors per lane (3072 bf16 columns, the Flux hidden size) get the unrolled form.
  constexpr int kUnrolled = 12;
  auto kern = cols == kUnrolled * 32 * Vec<T>::N ? norm_rows_bulk_kernel<T, kLayerNorm, kStagedMod, kUnrolled>
                                                 : norm_rows_bulk_kernel<T, kLayerNorm, kStagedMod, 0>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess)
    return set_error(FLUXB_ERR_CUDA, "row norm: cannot set shared memory size: %s", cudaGetErrorString(e));
  kern<<<(unsigned)((rows + warps - 1) / warps), warps * 32, smem, st>>>(
      x, scale, shift, y, rstd, rows, (int)cols, rpb, xaddr, y_ld, mod_stride, eps, device_status_ptr());
  return FLUXB_OK;
}

// Rows of up to 6 KB whose blocks of 16 rows each stay inside one batch element, with 16-byte
// aligned per-column vectors, take the form that stages those vectors in shared memory.
template <typename T, bool kLayerNorm>
static int launch_norm_bulk(const T* x, const T* scale, const T* shift, T* y, float* rstd, int64_t rows,
                            int64_t cols, int64_t rpb, RowAddr xaddr, int64_t y_ld, int64_t mod_stride, float eps,
                            cudaStream_t st) {
  const bool aligned = (reinterpret_cast<uintptr_t>(scale) & 15) == 0 &&
                       (!kLayerNorm || ((reinterpret_cast<uintptr_t>(shift) & 15) == 0 &&
                                        (mod_stride * (int64_t)sizeof(T)) % 16 == 0));
  const bool one_batch_per_block = !kLayerNorm || rpb % 16 == 0 || rows <= rpb;
  if (cols * (int64_t)sizeof(T) <= 6144 && aligned && one_batch_per_block)
    return launch_norm_bulk_as<T, kLayerNorm, true>(x, scale, shift, y, rstd, rows, cols, rpb, xaddr, y_ld,
                                                    mod_stride, eps, st);
  return launch_norm_bulk_as<T, kLayerNorm, false>(x, scale, shift, y, rstd, rows, cols, rpb, xaddr, y_ld,
                                                   mod_stride, eps, st);
}

template <typename T>
static int launch_ln_mod(const void* x, const void* scale, const void* shift, void* y, int64_t rows,
                         int64_t cols, int64_t rpb, int64_t x_ld, int64_t y_ld, int64_t mod_stride,
                         float eps, cudaStream_t st) {
  constexpr int VN = Vec<T>::N;
  const T* xp = static_cast<const T*>(x);
  const T* sc = static_cast<const T*>(scale);
  const T* sh = static_cast<const T*>(shift);
  T* yp = static_cast<T*>(y);
  const int64_t vecs = cols / VN;
  {
    RowAddr xaddr{1, rows > 0 ? rows : 1, 0, 0, x_ld, 1};
    if (bulk_rows_ok(cols, sizeof(T), xaddr) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      return launch_norm_bulk<T, true>(xp, sc, sh, yp, nullptr, rows, cols, rpb, xaddr, y_ld, mod_stride, eps, st);
    }
  }
#define FLUXB_LN_CASE(G, VPL)                                                                  \
  if (vecs == (G) * (VPL)) {                                                                   \
    const int64_t gpb = 256 / (G);                                                             \
    ln_mod_rows_kernel<T, G, VPL><<<(unsigned)((rows + gpb - 1) / gpb), 256, 0, st>>>(         \
        xp, sc, sh, yp, rows, (int)cols, rpb, x_ld, y_ld, mod_stride, eps);                    \
    return FLUXB_OK;                                                                           \
  }
  FLUXB_LN_CASE(32, 1) FLUXB_LN_CASE(32, 2) FLUXB_LN_CASE(32, 3) FLUXB_LN_CASE(32, 4)
  FLUXB_LN_CASE(32, 6) FLUXB_LN_CASE(32, 8) FLUXB_LN_CASE(32, 12) FLUXB_LN_CASE(32, 16)
  FLUXB_LN_CASE(32, 24)
#undef FLUXB_LN_CASE
  ln_mod_generic_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
      xp, sc, sh, yp, rows, (int)cols, rpb, x_ld, y_ld, mod_stride, eps);
  return FLUXB_OK;
}

// ----------------------------------------------------------------------------------------
// RMSNorm forward.  Input rows addressed through a 3-level stride (head-split views).
// ----------------------------------------------------------------------------------------

template <typename T, int G, int VPL>
__global__ void __launch_bounds__(256, (VPL <= 12 ? 3 : (VPL <= 24 ? 2 : 1)))
rms_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                float* __restrict__ rstd_out, int64_t rows, int cols, RowAddr addr, float eps) {
  constexpr int VN = Vec<T>::N;
  const int lig = threadIdx.x % G;
  const int64_t gpb = blockDim.x / G;
  const int64_t row = blockIdx.x * gpb + threadIdx.x / G;
  const bool active = row < rows;
  const int64_t r = active ? row : rows - 1;
  const T* xr = x + addr.offset(r);
  uint4 raw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) raw[i] = *reinterpret_cast<const uint4*>(xr + (i * G + lig) * VN);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    Vec<T> t;
    t.unpack(raw[i]);
#pragma unroll
    for (int j = 0; j < VN; ++j) s += t.v[j] * t.v[j];
  }
  const float rstd = rsqrtf(group_sum<G>(s) / cols + eps);
  if (active && rstd_out != nullptr && lig == 0) rstd_out[r] = rstd;
  T* yr = y + r * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * G + lig) * VN;
    Vec<T> t, wv;
    forget(raw[i]);
    t.unpack(raw[i]);
    wv.load_nc(w + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) t.v[j] = t.v[j] * rstd * wv.v[j];
    if (active) t.store(yr + c);
  }
}

// Narrow rows (one 16-byte vector per lane, e.g. the 128-wide per-head rows of q and k): a
// group of G lanes walks R rows with all R loads issued before the first reduction, so that a
// thread has R x 16 bytes in flight instead of 16.  Small blocks at high occupancy (128 threads,
// 12 blocks per SM: 96 KB in flight per SM) measured fastest: blocks retire and start
// continuously, so loads and stores of different blocks overlap throughout the launch.
template <typename T, int G, int R>
__global__ void __launch_bounds__(128, 12)
rms_narrow_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                       float* __restrict__ rstd_out, int64_t rows, int cols, RowAddr addr, float eps) {
  constexpr int VN = Vec<T>::N;
  const int lig = threadIdx.x % G;
  const int64_t gpb = blockDim.x / G;
  const int64_t row0 = (blockIdx.x * gpb + threadIdx.x / G) * R;
  uint4 raw[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int64_t r = row0 + i < rows ? row0 + i : rows - 1;
    raw[i] = ld_nc_u4(x + addr.offset(r) + lig * VN);
  }
  Vec<T> wv;
  wv.load_nc(w + lig * VN);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    Vec<T> t;
    t.unpack(raw[i]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < VN; ++j) s += t.v[j] * t.v[j];
    const float rstd = rsqrtf(group_sum<G>(s) / cols + eps);
    const int64_t r = row0 + i;
    if (r < rows) {
      if (rstd_out != nullptr && lig == 0) rstd_out[r] = rstd;
#pragma unroll
      for (int j = 0; j < VN; ++j) t.v[j] = t.v[j] * rstd * wv.v[j];
      t.store(y + r * (int64_t)cols + lig * VN);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
rms_generic_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                   float* __restrict__ rstd_out, int64_t rows, int cols, RowAddr addr, float eps) {
  constexpr int VN = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const T* xr = x + addr.offset(row);
  float s = 0.f;
  for (int c = lane * VN; c < cols; c += 32 * VN) {
    Vec<T> t;
    t.load(xr + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) s += t.v[j] * t.v[j];
  }
  const float rstd = rsqrtf(warp_sum(s) / cols + eps);
  if (rstd_out != nullptr && lane == 0) rstd_out[row] = rstd;
  T* yr = y + row * (int64_t)cols;
  for (int c = lane * VN; c < cols; c += 32 * VN) {
    Vec<T> t, wv;
    t.load(xr + c);
    wv.load_nc(w + c);
#pragma unroll
    for (int j = 0; j < VN; ++j) t.v[j] = t.v[j] * rstd * wv.v[j];
    t.store(yr + c);
  }
}

template <typename T>
static int launch_rms(const void* x, const void* w, void* y, float* rstd, int64_t rows, int64_t cols,
                      RowAddr addr, float eps, cudaStream_t st) {
  constexpr int VN = Vec<T>::N;
  const T* xp = static_cast<const T*>(x);
  const T* wp = static_cast<const T*>(w);
  T* yp = static_cast<T*>(y);
  const int64_t vecs = cols / VN;
  if (bulk_rows_ok(cols, sizeof(T), addr) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    return launch_norm_bulk<T, false>(xp, wp, nullptr, yp, rstd, rows, cols, 1, addr, cols, 0, eps, st);
  }
#define FLUXB_RMS_CASE(G, VPL)                                                                 \
  if (vecs == (G) * (VPL)) {                                                                   \
    const int64_t gpb = 256 / (G);                                                             \
    rms_rows_kernel<T, G, VPL><<<(unsigned)((rows + gpb - 1) / gpb), 256, 0, st>>>(            \
        xp, wp, yp, rstd, rows, (int)cols, addr, eps);                                         \
    return FLUXB_OK;                                                                           \
  }
#define FLUXB_RMS_NARROW(G)                                                                    \
  if (vecs == (G)) {                                                                           \
    const int64_t rpb = (128 / (G)) * 4;                                                       \
    rms_narrow_rows_kernel<T, G, 4><<<(unsigned)((rows + rpb - 1) / rpb), 128, 0, st>>>(       \
        xp, wp, yp, rstd, rows, (int)cols, addr, eps);                                         \
    return FLUXB_OK;                                                                           \
  }
  FLUXB_RMS_NARROW(8) FLUXB_RMS_NARROW(16) FLUXB_RMS_NARROW(32)
#undef FLUXB_RMS_NARROW
  FLUXB_RMS_CASE(32, 2)
  FLUXB_RMS_CASE(32, 3) FLUXB_RMS_CASE(32, 4) FLUXB_RMS_CASE(32, 6) FLUXB_RMS_CASE(32, 8)
  FLUXB_RMS_CASE(32, 12) FLUXB_RMS_CASE(32, 16) FLUXB_RMS_CASE(32, 24)
#undef FLUXB_RMS_CASE
  rms_generic_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(xp, wp, yp, rstd, rows,
                                                                    (int)cols, addr, eps);
  return FLUXB_OK;
}

// ----------------------------------------------------------------------------------------
// RMSNorm backward.  One warp per row for dx; each block also accumulates its rows' dw
// contributions in registers and writes one fp32 partial row per block (no atomics, so the
// result is deterministic); the caller sums the partial rows.
// ----------------------------------------------------------------------------------------
constexpr int kRmsBwdRowsPerBlock = 64;

template <typename T>
__global__ void __launch_bounds__(256)
rms_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
               const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial,
               int64_t rows, int cols) {
  constexpr int VN = Vec<T>::N;
  extern __shared__ float dw_smem[];  // [8 warps][cols]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float* my_dw = dw_smem + (int64_t)warp * cols;
  for (int c = lane; c < cols; c += 32) my_dw[c] = 0.f;
  __syncwarp();
  const int64_t row0 = (int64_t)blockIdx.x * kRmsBwdRowsPerBlock;
  for (int rr = warp; rr < kRmsBwdRowsPerBlock; rr += 8) {
    const int64_t row = row0 + rr;
    if (row >= rows) break;
    const T* dyr = dy + row * (int64_t)cols;
    const T* xr = x + row * (int64_t)cols;
    const float rs = rstd[row];
    float dot = 0.f;
    for (int c = lane * VN; c < cols; c += 32 * VN) {
      Vec<T> a, b, ww;
      a.load(dyr + c);
      b.load(xr + c);
      ww.load_nc(w + c);
#pragma unroll
      for (int j = 0; j < VN; ++j) dot += a.v[j] * ww.v[j] * b.v[j];
    }
    dot = warp_sum(dot);
    const float coef = -rs * rs * rs * dot / cols;
    T* dxr = dx + row * (int64_t)cols;
    for (int c = lane * VN; c < cols; c += 32 * VN) {
      Vec<T> a, b, ww, o;
      a.load(dyr + c);
      b.load(xr + c);
      ww.load_nc(w + c);
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        o.v[j] = rs * a.v[j] * ww.v[j] + coef * b.v[j];
        my_dw[c + j] += a.v[j] * b.v[j] * rs;
      }
      o.store(dxr + c);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) s += dw_smem[(int64_t)wi * cols + c];
    dw_partial[(int64_t)blockIdx.x * cols + c] = s;
  }
}

// ----------------------------------------------------------------------------------------
// RMSNorm backward without any allocation: the per-block partial sums of dw go to a fixed
// array that is part of the library image instead of caller-provided scratch.
//
// The array lives in device global memory of every GPU that loads the library, from load
// until the process exits (4 MiB per GPU).  Its name is only a handle in host code — it is
// not a device address there — so the host resolves the real address once per device with
// cudaGetSymbolAddress (see static_dw_scratch below) and passes that pointer to the kernels.
// ----------------------------------------------------------------------------------------
constexpr int64_t kStaticDwScratchFloats = 1 << 20;  // 1 Mi floats = 4 MiB
static __device__ __align__(256) float g_static_dw_scratch[kStaticDwScratchFloats];

// dw[c] = sum over the `parts` partial rows; one thread per column, fixed order (deterministic).
__global__ void __launch_bounds__(256)
reduce_dw_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw, int parts, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = 0; r < parts; ++r) s += partial[(int64_t)r * cols + c];
  dw[c] = s;
}

// ----------------------------------------------------------------------------------------
// RoPE with a general 2x2 table.  A thread owns 4 pairs (8 bf16 / 2x4 fp32) of one token and
// walks HG heads with the table entries held in registers.
// ----------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  Vec<__nv_bfloat16> t;
  t.load(p);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = t.v[j];
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 t;
  t.x = pack_bf16(v[0], v[1]); t.y = pack_bf16(v[2], v[3]);
  t.z = pack_bf16(v[4], v[5]); t.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = t;
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// f[i] = {f00, f01, f10, f11} for pair i;  out[2i] = f00 x0 + f01 x1, out[2i+1] = f10 x0 + f11 x1
__device__ __forceinline__ void rotate8(const float4 (&f)[4], const float (&x)[8], float (&o)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = f[i].x * x[2 * i] + f[i].y * x[2 * i + 1];
    o[2 * i + 1] = f[i].z * x[2 * i] + f[i].w * x[2 * i + 1];
  }
}

template <typename T, int HG>
__global__ void __launch_bounds__(256)
rope_kernel(const T* __restrict__ q, const T* __restrict__ k, const float* __restrict__ pe,
            T* __restrict__ oq, T* __restrict__ ok, int64_t BH, int64_t L, int D) {
  const int chunks = D / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= L * chunks) return;
  const int64_t l = idx / chunks;
  const int c = (int)(idx % chunks);
  float4 f[4];
  const float4* pr = reinterpret_cast<const float4*>(pe) + l * (D / 2) + c * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __ldg(pr + i);
  const int64_t bh0 = (int64_t)blockIdx.y * HG;
  const int64_t off0 = l * D + c * 8;
  float xq[HG][8], xk[HG][8];
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    if (bh0 + h < BH) {
      load8<T>(q + (bh0 + h) * L * D + off0, xq[h]);
      load8<T>(k + (bh0 + h) * L * D + off0, xk[h]);
    }
  }
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    if (bh0 + h < BH) {
      float o[8];
      rotate8(f, xq[h], o);
      store8<T>(oq + (bh0 + h) * L * D + off0, o);
      rotate8(f, xk[h], o);
      store8<T>(ok + (bh0 + h) * L * D + off0, o);
    }
  }
}

// bf16 form: the 16-byte pieces stay packed until they are rotated, so HG heads of q and k in
// flight cost 8 x HG registers instead of 16 x HG, and small blocks keep many of them resident.
template <int HG, int TPB, int MINB>
__global__ void __launch_bounds__(TPB, MINB)
rope_bf16_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                 const float* __restrict__ pe, __nv_bfloat16* __restrict__ oq, __nv_bfloat16* __restrict__ ok,
                 int BH, int64_t L, int D) {
  const int chunks = D / 8;
  const int64_t idx = (int64_t)blockIdx.x * TPB + threadIdx.x;
  if (idx >= L * chunks) return;
  const int64_t l = idx / chunks;
  const int c = (int)(idx % chunks);
  const int bh0 = blockIdx.y * HG;
  const int64_t off0 = l * D + c * 8;
  const int64_t head = L * D;
  uint4 rq[HG], rk[HG];
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    const int bh = bh0 + h < BH ? bh0 + h : BH - 1;
    rq[h] = ld_nc_u4(q + bh * head + off0);
    rk[h] = ld_nc_u4(k + bh * head + off0);
  }
  float4 f[4];
  const float4* pr = reinterpret_cast<const float4*>(pe) + l * (D / 2) + c * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __ldg(pr + i);
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    if (bh0 + h < BH) {
      Vec<__nv_bfloat16> t;
      float o[8];
      t.unpack(rq[h]);
      rotate8(f, t.v, o);
      store8<__nv_bfloat16>(oq + (bh0 + h) * head + off0, o);
      t.unpack(rk[h]);
      rotate8(f, t.v, o);
      store8<__nv_bfloat16>(ok + (bh0 + h) * head + off0, o);
    }
  }
}

// ----------------------------------------------------------------------------------------
// Fused q/k/v assembly: split + per-head RMSNorm of q,k + RoPE + head-major concat of up to
// two token streams.  16 lanes own one (token, head) row of 128; a thread walks HG heads of
// its token with the rope entries in registers.  bf16 only, D = 128.
// ----------------------------------------------------------------------------------------
struct QkvPrepArgs {
  const __nv_bfloat16* src[2];
  int64_t len[2];
  int64_t ld[2];
  const __nv_bfloat16* qscale[2];
  const __nv_bfloat16* kscale[2];
  const float* pe;
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  int64_t B, H, L;
  // output addressing: element offset = b*o_sb + (h / hpg)*o_sg + (h % hpg)*o_sh + l*o_sl
  int64_t o_sb, o_sg, o_sh, o_sl, hpg;
  float eps;
  // Scatter form (n_gbase > 0): head group g goes to gbase[g] (q), gbase[g] + k_off (k) and
  // gbase[g] + v_off (v) instead of q/k/v + g*o_sg; the bases may be other GPUs' memory.
  int n_gbase;
  int64_t k_off, v_off;
  __nv_bfloat16* gbase[8];
};

template <int HG, int TPB, int MINB>
__global__ void __launch_bounds__(TPB, MINB) qkv_prep_kernel(QkvPrepArgs a) {
  constexpr int D = 128;
  const int lane16 = threadIdx.x & 15;
  // Plain form: blockIdx.x walks token blocks, blockIdx.y head blocks.  Scatter form: the other
  // way round, so that blocks that run at the same time write to different destinations (local
  // memory and every peer) instead of one destination after the other.
  const unsigned tok_blk = a.n_gbase > 0 ? blockIdx.y : blockIdx.x;
  const unsigned head_blk = a.n_gbase > 0 ? blockIdx.x : blockIdx.y;
  const int64_t tok = (int64_t)tok_blk * (TPB / 16) + threadIdx.x / 16;  // b * L + l
  const bool active = tok < a.B * a.L;
  const int64_t t = active ? tok : a.B * a.L - 1;
  // Heads, heads per group and the sequence length fit 32 bits (the launcher checks): the
  // divisions below would otherwise cost more than the row's arithmetic.
  const int Li = (int)a.L, Hi = (int)a.H, hpg = (int)a.hpg;
  const int b = (int)(t / Li);
  const int l = (int)(t - (int64_t)b * Li);
  const int s = (l < a.len[0]) ? 0 : 1;
  const int64_t ls = (s == 0) ? l : l - a.len[0];
  const __nv_bfloat16* row = a.src[s] + (b * a.len[s] + ls) * a.ld[s];
  const int64_t HD = (int64_t)Hi * D;

  const int h0 = (int)head_blk * HG;
  uint4 raw[HG][3];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    const int h = h0 + hh < Hi ? h0 + hh : Hi - 1;
#pragma unroll
    for (int part = 0; part < 3; ++part) raw[hh][part] = ld_nc_u4(row + part * HD + h * D + lane16 * 8);
  }
  float4 f[4];
  const bool do_rope = a.pe != nullptr;
  if (do_rope) {
    const float4* pr = reinterpret_cast<const float4*>(a.pe) + (int64_t)l * (D / 2) + lane16 * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __ldg(pr + i);
  }
  const bool do_norm = a.qscale[s] != nullptr;
  uint4 wraw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};  // q and k weights, packed
  if (do_norm) {
    wraw[0] = ld_nc_u4(a.qscale[s] + lane16 * 8);
    wraw[1] = ld_nc_u4(a.kscale[s] + lane16 * 8);
  }
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    const int h = h0 + hh;
    if (h >= Hi) continue;  // uniform across the block (depends on the head block only)
    const int grp = h / hpg;
    int64_t out_off = b * a.o_sb + (h - grp * hpg) * a.o_sh + l * a.o_sl + lane16 * 8;
    __nv_bfloat16* qk_base[2] = {a.q, a.k};
    __nv_bfloat16* v_base = a.v;
    if (a.n_gbase > 0) {
      __nv_bfloat16* gb = a.gbase[grp];
      qk_base[0] = gb;
      qk_base[1] = gb + a.k_off;
      v_base = gb + a.v_off;
    } else {
      out_off += grp * a.o_sg;
    }
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      Vec<__nv_bfloat16> xv;
      xv.unpack(raw[hh][part]);
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = xv.v[j];
      if (do_norm) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
        const float rstd = rsqrtf(group_sum<16>(ss) / D + a.eps);
        Vec<__nv_bfloat16> wsel;
        wsel.unpack(wraw[part]);
        // Normalised values stay in fp32 through the rotation: one rounding, at the store.
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = x[j] * rstd * wsel.v[j];
      }
      float o[8];
      if (do_rope) {
        rotate8(f, x, o);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = x[j];
      }
      if (active) store8<__nv_bfloat16>(qk_base[part] + out_off, o);
    }
    if (active) *reinterpret_cast<uint4*>(v_base + out_off) = raw[hh][2];
  }
}

// ----------------------------------------------------------------------------------------
// Elementwise modulation kernels and SiLU.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
mod_scale_shift_kernel(const T* __restrict__ x, const T* __restrict__ mod, T* __restrict__ out,
                       int64_t nvec, int64_t L, int C, int64_t mod_row_stride, int shift_chunk,
                       int scale_chunk) {
  constexpr int VN = Vec<T>::N;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const int64_t e = i * VN;
  const int c = (int)(e % C);
  const int64_t b = e / ((int64_t)C * L);
  Vec<T> xv, sc, sh;
  xv.load(x + e);
  sh.load_nc(mod + b * mod_row_stride + (int64_t)shift_chunk * C + c);
  sc.load_nc(mod + b * mod_row_stride + (int64_t)scale_chunk * C + c);
#pragma unroll
  for (int j = 0; j < VN; ++j) xv.v[j] = (sc.v[j] + 1.0f) * xv.v[j] + sh.v[j];
  xv.store(out + e);
}

template <typename T>
__global__ void __launch_bounds__(256)
mod_gate_proj_kernel(const T* __restrict__ resid, const T* __restrict__ mod,
                     const T* __restrict__ proj, T* __restrict__ out, int64_t nvec, int64_t L, int C,
                     int64_t mod_row_stride, int gate_chunk) {
  constexpr int VN = Vec<T>::N;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const int64_t e = i * VN;
  const int c = (int)(e % C);
  const int64_t b = e / ((int64_t)C * L);
  Vec<T> r, p, g;
  r.load(resid + e);
  p.load(proj + e);
  g.load_nc(mod + b * mod_row_stride + (int64_t)gate_chunk * C + c);
#pragma unroll
  for (int j = 0; j < VN; ++j) r.v[j] = r.v[j] + g.v[j] * p.v[j];
  r.store(out + e);
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n) {
  constexpr int VN = Vec<T>::N;
  const int64_t e = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VN;
  if (e + VN <= n) {
    Vec<T> v;
    v.load(x + e);
#pragma unroll
    for (int j = 0; j < VN; ++j) v.v[j] = silu_f(v.v[j]);
    v.store(out + e);
  } else {
    for (int64_t i = e; i < n; ++i) out[i] = static_cast<T>(silu_f(static_cast<float>(x[i])));
  }
}

// ----------------------------------------------------------------------------------------
// Modulation projection, rows of whole 1536-element chunks (the Flux hidden size is two).
//
// The kernel is a 113 MB weight stream (double-stream block) that has to run at HBM speed, so the
// per-byte work of a lane is kept to almost nothing:
//  * act(vec) is staged in shared memory as bf16 (the reference's SiLU output is bf16 too) and the
//    products run on the tensor pipe.  A lane's 16-byte weight load is used AS an mma A fragment
//    (registers a0..a3 = the four words): word 0/2 sit in fragment row g = lane/4, word 1/3 in row
//    g+8.  The B fragment of the same lane (column g) is given the activations at the same k
//    positions as its own weight words, so the diagonal D[g][g] of mma #1 (B from words 0,2) and
//    D[g+8][g] of mma #2 (B from words 1,3) accumulate exactly that lane group's products.  The row
//    result is the sum of the diagonals over the warp.  Two mma per 16-byte load replace eight
//    unpacks, eight multiply-adds and 32 bytes of shared-memory reads.
//  * vec is requested before any weight (a request behind the weight stream comes back last), and
//    half-row chunks of six loads per lane are double-buffered across row boundaries.
//  * the grid is balanced: every warp gets the same number of rows when N allows it.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

template <int BT>
__global__ void __launch_bounds__(512, 2)
mod_gemv_mma_kernel(const __nv_bfloat16* __restrict__ vec, const __nv_bfloat16* __restrict__ w,
                    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int64_t N,
                    int K, int64_t b0, int apply_silu, int64_t out_stride) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  __nv_bfloat16* sa = reinterpret_cast<__nv_bfloat16*>(gemv_smem);  // act(vec) [BT][K]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int cpr = K / 1536;
  // rows are counted in 32 bits (the launcher checks N): 64-bit row arithmetic costs registers
  const int n_rows = (int)N;
  const int stride = gridDim.x * warps;
  int row = blockIdx.x * warps + warp;
  // vec first
  const int nv = BT * K / 8;
  constexpr int kVecRegs = 1;  // one 16-byte piece per thread (512 threads cover BT x K up to 4096 elements)
  uint4 myvec[kVecRegs];
  const int nthr = blockDim.x;
#pragma unroll
  for (int r = 0; r < kVecRegs; ++r) {
    const int i = threadIdx.x + r * nthr;
    if (i < nv) myvec[r] = ld_nc_u4(vec + b0 * K + (int64_t)i * 8);
  }
  uint4 cur[6], nxt[6];
  if (row < n_rows) {
#pragma unroll
    for (int u = 0; u < 6; ++u) cur[u] = ld_nc_u4(w + (int64_t)row * K + lane * 8 + u * 256);
  }
  auto stage = [&](const uint4& raw, int i) {
    Vec<__nv_bfloat16> t;
    t.unpack(raw);
    if (apply_silu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) t.v[j] = silu_f(t.v[j]);
    }
    t.store(sa + (int64_t)i * 8);
  };
#pragma unroll
  for (int r = 0; r < kVecRegs; ++r) {
    const int i = threadIdx.x + r * nthr;
    if (i < nv) stage(myvec[r], i);
  }
  for (int i = threadIdx.x + kVecRegs * nthr; i < nv; i += nthr) stage(ld_nc_u4(vec + b0 * K + (int64_t)i * 8), i);
  __syncthreads();

  float c1[BT][4], c2[BT][4];
#pragma unroll
  for (int bb = 0; bb < BT; ++bb)
#pragma unroll
    for (int j = 0; j < 4; ++j) c1[bb][j] = c2[bb][j] = 0.f;
  const int g = lane >> 2;
  const bool on_diagonal = (lane & 3) == (g >> 1);
  int ch = 0;
  while (row < n_rows) {
    const bool last = ch + 1 == cpr;
    const int nrow = last ? row + stride : row;
    const int nch = last ? 0 : ch + 1;
    if (nrow < n_rows) {
#pragma unroll
      for (int u = 0; u < 6; ++u) nxt[u] = ld_nc_u4(w + (int64_t)nrow * K + nch * 1536 + lane * 8 + u * 256);
    }
    const __nv_bfloat16* sac = sa + ch * 1536 + lane * 8;
#pragma unroll
    for (int u = 0; u < 6; ++u) {
#pragma unroll
      for (int bb = 0; bb < BT; ++bb) {
        const uint4 a = *reinterpret_cast<const uint4*>(sac + bb * K + u * 256);
        mma_bf16_16x8x16(c1[bb], cur[u], a.x, a.z);
        mma_bf16_16x8x16(c2[bb], cur[u], a.y, a.w);
      }
    }
    if (last) {
#pragma unroll
      for (int bb = 0; bb < BT; ++bb) {
        const float mine = on_diagonal ? ((g & 1) ? c1[bb][1] + c2[bb][3] : c1[bb][0] + c2[bb][2]) : 0.f;
        const float sum = warp_sum(mine);
        if (lane == 0) {
          const float bv = bias != nullptr ? __bfloat162float(bias[row]) : 0.f;
          out[(b0 + bb) * out_stride + row] = __float2bfloat16_rn(sum + bv);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) c1[bb][j] = c2[bb][j] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 6; ++u) cur[u] = nxt[u];
    row = nrow;
    ch = nch;
  }
}

// ----------------------------------------------------------------------------------------
// Modulation projection: out[b,n] = sum_k act(vec[b,k]) w[n,k] + bias[n], bf16 weights read
// exactly once per batch tile of BT rows.  One warp per output column n; act(vec) staged in
// shared memory as fp32.
// ----------------------------------------------------------------------------------------
template <int BT>
__global__ void __launch_bounds__(512, 2)
mod_gemv_kernel(const __nv_bfloat16* __restrict__ vec, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int64_t N,
                int K, int64_t b0, int apply_silu, int64_t out_stride) {
  extern __shared__ float sv[];  // [BT][K]
  for (int i = threadIdx.x; i < BT * K; i += blockDim.x) {
    const int bb = i / K, kk = i % K;
    float t = __bfloat162float(vec[(b0 + bb) * K + kk]);
    if (apply_silu) t = silu_f(t);  // kept in fp32: no intermediate rounding
    sv[i] = t;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  // A few persistent blocks per SM; every warp walks output columns with a grid stride.
  for (int64_t n = (int64_t)blockIdx.x * warps + warp; n < N; n += (int64_t)gridDim.x * warps) {
    const __nv_bfloat16* wr = w + n * K;
    float acc[BT];
#pragma unroll
    for (int bb = 0; bb < BT; ++bb) acc[bb] = 0.f;
    int k0 = lane * 8;
    // Whole 3072-wide rows (the Flux hidden size) are fetched with all twelve 16-byte loads of a
    // lane in flight at once; other widths go four loads at a time.
    for (; k0 + 11 * 256 < K; k0 += 12 * 256) {
      uint4 raw[12];
#pragma unroll
      for (int u = 0; u < 12; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(wr + k0 + u * 256));
      // pin the schedule: all twelve loads are issued before the first value is consumed
#pragma unroll
      for (int u = 0; u < 12; ++u) forget(raw[u]);
#pragma unroll
      for (int u = 0; u < 12; ++u) {
        Vec<__nv_bfloat16> wv;
        wv.unpack(raw[u]);
#pragma unroll
        for (int bb = 0; bb < BT; ++bb) {
          const float4 a0 = *reinterpret_cast<const float4*>(sv + bb * K + k0 + u * 256);
          const float4 a1 = *reinterpret_cast<const float4*>(sv + bb * K + k0 + u * 256 + 4);
          acc[bb] += wv.v[0] * a0.x + wv.v[1] * a0.y + wv.v[2] * a0.z + wv.v[3] * a0.w +
                     wv.v[4] * a1.x + wv.v[5] * a1.y + wv.v[6] * a1.z + wv.v[7] * a1.w;
        }
      }
    }
    for (; k0 + 3 * 256 < K; k0 += 4 * 256) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(wr + k0 + u * 256));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        Vec<__nv_bfloat16> wv;
        wv.unpack(raw[u]);
#pragma unroll
        for (int bb = 0; bb < BT; ++bb) {
          const float4 a0 = *reinterpret_cast<const float4*>(sv + bb * K + k0 + u * 256);
          const float4 a1 = *reinterpret_cast<const float4*>(sv + bb * K + k0 + u * 256 + 4);
          acc[bb] += wv.v[0] * a0.x + wv.v[1] * a0.y + wv.v[2] * a0.z + wv.v[3] * a0.w +
                     wv.v[4] * a1.x + wv.v[5] * a1.y + wv.v[6] * a1.z + wv.v[7] * a1.w;
        }
      }
    }
    for (; k0 < K; k0 += 256) {
      Vec<__nv_bfloat16> wv;
      wv.load_nc(wr + k0);
#pragma unroll
      for (int bb = 0; bb < BT; ++bb) {
        const float4 a0 = *reinterpret_cast<const float4*>(sv + bb * K + k0);
        const float4 a1 = *reinterpret_cast<const float4*>(sv + bb * K + k0 + 4);
        acc[bb] += wv.v[0] * a0.x + wv.v[1] * a0.y + wv.v[2] * a0.z + wv.v[3] * a0.w +
                   wv.v[4] * a1.x + wv.v[5] * a1.y + wv.v[6] * a1.z + wv.v[7] * a1.w;
      }
    }
#pragma unroll
    for (int bb = 0; bb < BT; ++bb) {
      const float s = warp_sum(acc[bb]);
      if (lane == 0) {
        const float bv = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
        out[(b0 + bb) * out_stride + n] = __float2bfloat16_rn(s + bv);
      }
    }
  }
}

}  // namespace fluxb

// ========================================================================================
// C ABI
// ========================================================================================
using namespace fluxb;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return FLUXB_OK;
}
static inline int vec_elems(int dtype) { return dtype == FLUXB_BF16 ? 8 : 4; }

extern "C" int fluxb_layer_norm_modulation(const void* x, const void* scale, const void* shift,
                                           void* y, int64_t rows, int64_t cols,
                                           int64_t rows_per_batch, int64_t x_ld, int64_t y_ld,
                                           int64_t mod_stride, float eps, int dtype,
                                           fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "layer_norm_modulation: dtype %d", dtype);
  if (rows < 0 || cols <= 0 || rows_per_batch < 0)
    return set_error(FLUXB_ERR_BAD_ARG, "layer_norm_modulation: bad sizes");
  if (rows == 0) return FLUXB_OK;  // zero tokens (rows_per_batch is 0 then, too)
  if (rows_per_batch == 0) return set_error(FLUXB_ERR_BAD_ARG, "layer_norm_modulation: rows_per_batch is 0");
  if (!x || !scale || !shift || !y)
    return set_error(FLUXB_ERR_BAD_ARG, "layer_norm_modulation: null pointer");
  const int vn = vec_elems(dtype);
  if (cols % vn || x_ld % vn || y_ld % vn || mod_stride % vn || !aligned16(x) || !aligned16(y) ||
      !aligned16(scale) || !aligned16(shift))
    return set_error(FLUXB_ERR_BAD_ARG,
                     "layer_norm_modulation: cols/strides must be multiples of %d elements and "
                     "pointers 16-byte aligned", vn);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = dtype == FLUXB_BF16
                     ? launch_ln_mod<__nv_bfloat16>(x, scale, shift, y, rows, cols, rows_per_batch, x_ld, y_ld,
                                                    mod_stride, eps, st)
                     : launch_ln_mod<float>(x, scale, shift, y, rows, cols, rows_per_batch, x_ld, y_ld, mod_stride,
                                            eps, st);
  if (rc != FLUXB_OK) return rc;
  return launch_status("layer_norm_modulation");
}

extern "C" int fluxb_rms_norm(const void* x, const void* w, void* y, float* rstd, int64_t n0,
                              int64_t n1, int64_t n2, int64_t cols, int64_t s0, int64_t s1,
                              int64_t s2, float eps, int dtype, fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "rms_norm: dtype %d", dtype);
  if (n0 < 0 || n1 < 0 || n2 < 0 || cols <= 0) return set_error(FLUXB_ERR_BAD_ARG, "rms_norm: bad sizes");
  const int64_t rows = n0 * n1 * n2;
  if (rows == 0) return FLUXB_OK;
  if (!x || !w || !y) return set_error(FLUXB_ERR_BAD_ARG, "rms_norm: null pointer");
  const int vn = vec_elems(dtype);
  if (cols % vn || s0 % vn || s1 % vn || s2 % vn || !aligned16(x) || !aligned16(y) || !aligned16(w))
    return set_error(FLUXB_ERR_BAD_ARG,
                     "rms_norm: cols/strides must be multiples of %d elements and pointers 16-byte "
                     "aligned", vn);
  const int flat = (n1 == 1 || s1 == n2 * s2) && (n0 == 1 || s0 == n1 * n2 * s2);
  RowAddr addr{n1, n2, s0, s1, s2, flat};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = dtype == FLUXB_BF16 ? launch_rms<__nv_bfloat16>(x, w, y, rstd, rows, cols, addr, eps, st)
                                     : launch_rms<float>(x, w, y, rstd, rows, cols, addr, eps, st);
  if (rc != FLUXB_OK) return rc;
  return launch_status("rms_norm");
}

extern "C" int64_t fluxb_rms_norm_bwd_partial_rows(int64_t rows) {
  return rows <= 0 ? 0 : (rows + kRmsBwdRowsPerBlock - 1) / kRmsBwdRowsPerBlock;
}

extern "C" int fluxb_rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                  void* dx, float* dw_partial, int64_t rows, int64_t cols, int dtype,
                                  fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "rms_norm_bwd: dtype %d", dtype);
  if (rows < 0 || cols <= 0) return set_error(FLUXB_ERR_BAD_ARG, "rms_norm_bwd: bad sizes");
  if (rows == 0) return FLUXB_OK;
  if (!dy || !x || !w || !rstd || !dx || !dw_partial)
    return set_error(FLUXB_ERR_BAD_ARG, "rms_norm_bwd: null pointer");
  const int vn = vec_elems(dtype);
  if (cols % vn || !aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx))
    return set_error(FLUXB_ERR_BAD_ARG, "rms_norm_bwd: cols must be a multiple of %d, pointers 16-byte aligned", vn);
  const size_t smem = (size_t)8 * cols * sizeof(float);
  if (smem > 200 * 1024) return set_error(FLUXB_ERR_UNSUPPORTED, "rms_norm_bwd: cols %lld too large", (long long)cols);
  const unsigned grid = (unsigned)fluxb_rms_norm_bwd_partial_rows(rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FLUXB_BF16) {
    auto kern = rms_bwd_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                                  static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx),
                                  dw_partial, rows, (int)cols);
  } else {
    auto kern = rms_bwd_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, 256, smem, st>>>(static_cast<const float*>(dy), static_cast<const float*>(x),
                                  static_cast<const float*>(w), rstd, static_cast<float*>(dx), dw_partial,
                                  rows, (int)cols);
  }
  return launch_status("rms_norm_bwd");
}

// Address of g_static_dw_scratch on the current device, resolved on first use per device.
static float* static_dw_scratch(int* err) {
  static std::mutex mu;
  static float* ptrs[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *err = set_error(FLUXB_ERR_CUDA, "rms_norm_bwd_static: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_dw_scratch);  // needs `dev` current, which it is
    if (e != cudaSuccess || p == nullptr) {
      *err = set_error(FLUXB_ERR_CUDA, "rms_norm_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = static_cast<float*>(p);
  }
  return ptrs[dev];
}

extern "C" int fluxb_rms_norm_bwd_static_max_floats(void) { return (int)kStaticDwScratchFloats; }

extern "C" int fluxb_rms_norm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                         void* dx, float* dw, int64_t rows, int64_t cols, int dtype,
                                         fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "rms_norm_bwd_static: dtype %d", dtype);
  if (rows < 0 || cols <= 0) return set_error(FLUXB_ERR_BAD_ARG, "rms_norm_bwd_static: bad sizes");
  if (!dw) return set_error(FLUXB_ERR_BAD_ARG, "rms_norm_bwd_static: null dw");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaError_t e = cudaMemsetAsync(dw, 0, (size_t)cols * sizeof(float), st);
    if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "rms_norm_bwd_static: %s", cudaGetErrorString(e));
    return FLUXB_OK;
  }
  const int64_t parts = fluxb_rms_norm_bwd_partial_rows(rows);
  if (parts * cols > kStaticDwScratchFloats)
    return set_error(FLUXB_ERR_UNSUPPORTED,
                     "rms_norm_bwd_static: ceil(rows/%d) * cols = %lld floats of scratch needed, the built-in array "
                     "holds %lld; use fluxb_rms_norm_bwd with caller scratch",
                     kRmsBwdRowsPerBlock, (long long)(parts * cols), (long long)kStaticDwScratchFloats);
  int err = FLUXB_OK;
  float* scratch = static_dw_scratch(&err);
  if (scratch == nullptr) return err;
  // Stage 1: the ordinary backward kernel, writing its partial rows into the built-in array.
  // Every element of the region that stage 2 reads is overwritten here, so nothing left by an
  // earlier call can leak into this one and nothing needs clearing first.
  int rc = fluxb_rms_norm_bwd(dy, x, w, rstd, dx, scratch, rows, cols, dtype, stream);
  if (rc != FLUXB_OK) return rc;
  // Stage 2: fold the partial rows into the caller's dw.
  reduce_dw_partials_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, st>>>(scratch, dw, (int)parts, (int)cols);
  return launch_status("rms_norm_bwd_static");
}

extern "C" int fluxb_rope(const void* q, const void* k, const float* pe, void* oq, void* ok,
                          int64_t BH, int64_t L, int64_t D, int dtype, fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "rope: dtype %d", dtype);
  if (BH < 0 || L < 0 || D <= 0 || D % 8) return set_error(FLUXB_ERR_BAD_ARG, "rope: D must be a positive multiple of 8");
  if (BH == 0 || L == 0) return FLUXB_OK;
  if (!q || !k || !pe || !oq || !ok) return set_error(FLUXB_ERR_BAD_ARG, "rope: null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(pe) || !aligned16(oq) || !aligned16(ok))
    return set_error(FLUXB_ERR_BAD_ARG, "rope: pointers must be 16-byte aligned");
  constexpr int HG = 4;
  const int64_t threads = L * (D / 8);
  dim3 grid((unsigned)((threads + 255) / 256), (unsigned)((BH + HG - 1) / HG));
  if (grid.y > 65535) return set_error(FLUXB_ERR_UNSUPPORTED, "rope: batch*heads too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FLUXB_BF16) {
    // two heads of q and k per thread, 256-thread blocks at five per SM: fastest of a sweep over
    // 1-8 heads x 64-256 threads (19.5 us against 20.8 for one head, 20.4 for eight)
    constexpr int HGB = 2, TPB = 256;
    dim3 g2((unsigned)((threads + TPB - 1) / TPB), (unsigned)((BH + HGB - 1) / HGB));
    if (g2.y > 65535) return set_error(FLUXB_ERR_UNSUPPORTED, "rope: batch*heads too large");
    rope_bf16_kernel<HGB, TPB, 5><<<g2, TPB, 0, st>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), pe,
        static_cast<__nv_bfloat16*>(oq), static_cast<__nv_bfloat16*>(ok), (int)BH, L, (int)D);
  } else
    rope_kernel<float, HG><<<grid, 256, 0, st>>>(static_cast<const float*>(q),
                                                 static_cast<const float*>(k), pe,
                                                 static_cast<float*>(oq), static_cast<float*>(ok), BH,
                                                 L, (int)D);
  return launch_status("rope");
}

static int qkv_prep_impl(const void* src0, int64_t L0, int64_t ld0, const void* qscale0,
                         const void* kscale0, const void* src1, int64_t L1, int64_t ld1,
                         const void* qscale1, const void* kscale1, const float* pe, void* q,
                         void* k, void* v, int64_t B, int64_t H, int64_t D, int64_t heads_per_group,
                         int64_t o_sb, int64_t o_sg, int64_t o_sh, int64_t o_sl, float eps,
                         void* const* group_bases, int n_groups, int64_t k_off, int64_t v_off,
                         fluxb_stream_t stream) {
  if (D != 128) return set_error(FLUXB_ERR_UNSUPPORTED, "qkv_prep: head_dim %lld (only 128)", (long long)D);
  if (B < 0 || H <= 0 || L0 < 0 || L1 < 0) return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: bad sizes");
  const int64_t L = L0 + L1;
  if (B == 0 || L == 0) return FLUXB_OK;
  if ((n_groups == 0 && (!q || !k || !v)) || (L0 > 0 && !src0) || (L1 > 0 && !src1))
    return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: null pointer");
  if ((qscale0 == nullptr) != (kscale0 == nullptr) || (L1 > 0 && ((qscale1 == nullptr) != (kscale1 == nullptr))) ||
      (L0 > 0 && L1 > 0 && ((qscale0 == nullptr) != (qscale1 == nullptr))))
    return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: norm scales must be given for q and k of every stream or for none");
  if ((L0 > 0 && (ld0 < 3 * H * D || ld0 % 8)) || (L1 > 0 && (ld1 < 3 * H * D || ld1 % 8)))
    return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: row stride must be >= 3*H*D and a multiple of 8");
  if (!aligned16(src0) || !aligned16(src1) || !aligned16(q) || !aligned16(k) || !aligned16(v) ||
      !aligned16(pe) || !aligned16(qscale0) || !aligned16(kscale0) || !aligned16(qscale1) || !aligned16(kscale1))
    return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: pointers must be 16-byte aligned");
  QkvPrepArgs a;
  a.src[0] = static_cast<const __nv_bfloat16*>(src0);
  a.src[1] = static_cast<const __nv_bfloat16*>(src1);
  a.len[0] = L0; a.len[1] = L1;
  a.ld[0] = ld0; a.ld[1] = ld1;
  a.qscale[0] = static_cast<const __nv_bfloat16*>(qscale0);
  a.kscale[0] = static_cast<const __nv_bfloat16*>(kscale0);
  a.qscale[1] = static_cast<const __nv_bfloat16*>(qscale1);
  a.kscale[1] = static_cast<const __nv_bfloat16*>(kscale1);
  if (L0 == 0) {  // single stream given as stream 1: make it stream 0
    a.src[0] = a.src[1]; a.len[0] = L1; a.ld[0] = ld1; a.qscale[0] = a.qscale[1]; a.kscale[0] = a.kscale[1];
    a.len[1] = 0;
  }
  a.pe = pe;
  a.q = static_cast<__nv_bfloat16*>(q);
  a.k = static_cast<__nv_bfloat16*>(k);
  a.v = static_cast<__nv_bfloat16*>(v);
  a.B = B; a.H = H; a.L = L; a.eps = eps;
  a.n_gbase = 0; a.k_off = 0; a.v_off = 0;
  for (int i = 0; i < 8; ++i) a.gbase[i] = nullptr;
  if (n_groups > 0) {
    if (n_groups > 8 || heads_per_group <= 0 || heads_per_group * n_groups != H || !group_bases || k_off % 8 || v_off % 8)
      return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep_scatter: need 1..8 groups of heads_per_group heads covering H, and offsets that are multiples of 8");
    for (int i = 0; i < n_groups; ++i) {
      if (!group_bases[i] || !aligned16(group_bases[i]))
        return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep_scatter: group base %d is null or misaligned", i);
      a.gbase[i] = static_cast<__nv_bfloat16*>(group_bases[i]);
    }
    a.n_gbase = n_groups; a.k_off = k_off; a.v_off = v_off;
  }
  if (heads_per_group <= 0) {  // default: contiguous [B, H, L, D]
    a.hpg = H; a.o_sg = 0; a.o_sb = H * L * D; a.o_sh = L * D; a.o_sl = D;
  } else {
    if (H % heads_per_group || o_sb % 8 || o_sg % 8 || o_sh % 8 || o_sl % 8 || o_sl < D)
      return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep: heads_per_group must divide H and output strides must be multiples of 8 (row stride >= D)");
    a.hpg = heads_per_group; a.o_sg = o_sg; a.o_sb = o_sb; a.o_sh = o_sh; a.o_sl = o_sl;
  }
  if (H > 65535 || L > (int64_t)1 << 30 || heads_per_group > 65535)
    return set_error(FLUXB_ERR_UNSUPPORTED, "qkv_prep: H, heads per group <= 65535 and L <= 2^30");
  // Two heads per thread (six 16-byte loads in flight), 128-thread blocks at eight per SM:
  // fastest of a sweep over 1-4 heads x 128/256 threads (29.9 us against 34.2 for four heads in
  // 256-thread blocks at two per SM).
  constexpr int HG = 2, TPB = 128;
  dim3 grid((unsigned)((B * L + (TPB / 16) - 1) / (TPB / 16)), (unsigned)((H + HG - 1) / HG));
  if (a.n_gbase > 0) {
    if (grid.x > 65535) return set_error(FLUXB_ERR_UNSUPPORTED, "qkv_prep_scatter: more than 524280 tokens per call");
    grid = dim3(grid.y, grid.x);
  }
  qkv_prep_kernel<HG, TPB, 8><<<grid, TPB, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return launch_status("qkv_prep");
}

extern "C" int fluxb_qkv_prep(const void* src0, int64_t L0, int64_t ld0, const void* qscale0,
                              const void* kscale0, const void* src1, int64_t L1, int64_t ld1,
                              const void* qscale1, const void* kscale1, const float* pe, void* q,
                              void* k, void* v, int64_t B, int64_t H, int64_t D, int64_t heads_per_group,
                              int64_t o_sb, int64_t o_sg, int64_t o_sh, int64_t o_sl, float eps,
                              fluxb_stream_t stream) {
  return qkv_prep_impl(src0, L0, ld0, qscale0, kscale0, src1, L1, ld1, qscale1, kscale1, pe, q, k, v, B, H, D,
                       heads_per_group, o_sb, o_sg, o_sh, o_sl, eps, nullptr, 0, 0, 0, stream);
}

extern "C" int fluxb_qkv_prep_scatter(const void* src0, int64_t L0, int64_t ld0, const void* qscale0,
                                      const void* kscale0, const void* src1, int64_t L1, int64_t ld1,
                                      const void* qscale1, const void* kscale1, const float* pe,
                                      void* const* group_bases, int n_groups, int64_t k_off, int64_t v_off,
                                      int64_t B, int64_t H, int64_t D, int64_t heads_per_group, int64_t o_sb,
                                      int64_t o_sh, int64_t o_sl, float eps, fluxb_stream_t stream) {
  if (n_groups <= 0) return set_error(FLUXB_ERR_BAD_ARG, "qkv_prep_scatter: no groups");
  return qkv_prep_impl(src0, L0, ld0, qscale0, kscale0, src1, L1, ld1, qscale1, kscale1, pe, nullptr, nullptr,
                       nullptr, B, H, D, heads_per_group, o_sb, 0, o_sh, o_sl, eps, group_bases, n_groups, k_off,
                       v_off, stream);
}

template <typename T>
static void launch_scale_shift(const void* x, const void* mod, void* out, int64_t B, int64_t L,
                               int64_t C, int64_t mrs, int is_mod1, cudaStream_t st) {
  const int64_t nvec = B * L * C / Vec<T>::N;
  mod_scale_shift_kernel<T><<<(unsigned)((nvec + 255) / 256), 256, 0, st>>>(
      static_cast<const T*>(x), static_cast<const T*>(mod), static_cast<T*>(out), nvec, L, (int)C, mrs,
      is_mod1 ? 0 : 3, is_mod1 ? 1 : 4);
}

extern "C" int fluxb_modulation_scale_shift(const void* x, const void* mod, void* out, int64_t B,
                                            int64_t L, int64_t C, int64_t mod_row_stride,
                                            int is_mod1, int dtype, fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "modulation_scale_shift: dtype %d", dtype);
  if (B < 0 || L < 0 || C <= 0) return set_error(FLUXB_ERR_BAD_ARG, "modulation_scale_shift: bad sizes");
  if (B * L == 0) return FLUXB_OK;
  const int vn = vec_elems(dtype);
  if (!x || !mod || !out || C % vn || mod_row_stride % vn || !aligned16(x) || !aligned16(mod) || !aligned16(out))
    return set_error(FLUXB_ERR_BAD_ARG, "modulation_scale_shift: null/misaligned pointer or C not a multiple of %d", vn);
  if (mod_row_stride < (is_mod1 ? 2 : 5) * C)
    return set_error(FLUXB_ERR_BAD_ARG, "modulation_scale_shift: modulation row too short for the chunks asked");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FLUXB_BF16) launch_scale_shift<__nv_bfloat16>(x, mod, out, B, L, C, mod_row_stride, is_mod1, st);
  else launch_scale_shift<float>(x, mod, out, B, L, C, mod_row_stride, is_mod1, st);
  return launch_status("modulation_scale_shift");
}

template <typename T>
static void launch_gate_proj(const void* r, const void* mod, const void* p, void* out, int64_t B,
                             int64_t L, int64_t C, int64_t mrs, int chunk, cudaStream_t st) {
  const int64_t nvec = B * L * C / Vec<T>::N;
  mod_gate_proj_kernel<T><<<(unsigned)((nvec + 255) / 256), 256, 0, st>>>(
      static_cast<const T*>(r), static_cast<const T*>(mod), static_cast<const T*>(p),
      static_cast<T*>(out), nvec, L, (int)C, mrs, chunk);
}

extern "C" int fluxb_modulation_gate_proj(const void* resid, const void* mod, const void* proj,
                                          void* out, int64_t B, int64_t L, int64_t C,
                                          int64_t mod_row_stride, int gate_chunk, int dtype,
                                          fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16)
    return set_error(FLUXB_ERR_UNSUPPORTED, "modulation_gate_proj: dtype %d", dtype);
  if (B < 0 || L < 0 || C <= 0 || gate_chunk < 0) return set_error(FLUXB_ERR_BAD_ARG, "modulation_gate_proj: bad sizes");
  if (B * L == 0) return FLUXB_OK;
  const int vn = vec_elems(dtype);
  if (!resid || !mod || !proj || !out || C % vn || mod_row_stride % vn || !aligned16(resid) ||
      !aligned16(mod) || !aligned16(proj) || !aligned16(out))
    return set_error(FLUXB_ERR_BAD_ARG, "modulation_gate_proj: null/misaligned pointer or C not a multiple of %d", vn);
  if (mod_row_stride < (int64_t)(gate_chunk + 1) * C)
    return set_error(FLUXB_ERR_BAD_ARG, "modulation_gate_proj: modulation row too short for chunk %d", gate_chunk);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FLUXB_BF16) launch_gate_proj<__nv_bfloat16>(resid, mod, proj, out, B, L, C, mod_row_stride, gate_chunk, st);
  else launch_gate_proj<float>(resid, mod, proj, out, B, L, C, mod_row_stride, gate_chunk, st);
  return launch_status("modulation_gate_proj");
}

extern "C" int fluxb_silu(const void* x, void* out, int64_t n, int dtype, fluxb_stream_t stream) {
  if (dtype != FLUXB_F32 && dtype != FLUXB_BF16) return set_error(FLUXB_ERR_UNSUPPORTED, "silu: dtype %d", dtype);
  if (n < 0) return set_error(FLUXB_ERR_BAD_ARG, "silu: negative size");
  if (n == 0) return FLUXB_OK;
  if (!x || !out || !aligned16(x) || !aligned16(out)) return set_error(FLUXB_ERR_BAD_ARG, "silu: null or misaligned pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vn = vec_elems(dtype);
  const int64_t nvec = (n + vn - 1) / vn;
  const unsigned grid = (unsigned)((nvec + 255) / 256);
  if (dtype == FLUXB_BF16)
    silu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n);
  else
    silu_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out), n);
  return launch_status("silu");
}

// `light`: 128-thread blocks, at most two per SM: few enough registers, threads and shared memory
// to be resident beside a tensor-core kernel that holds one persistent block per SM, so that a
// projection whose result is needed later streams its weights while that kernel computes.
static int modulation_gemv_impl(const void* vec, const void* w, const void* bias, void* out, int64_t B,
                                int64_t N, int64_t K, int64_t out_stride, int apply_silu, bool light,
                                fluxb_stream_t stream) {
  if (B < 0 || N < 0 || K <= 0 || out_stride < N) return set_error(FLUXB_ERR_BAD_ARG, "modulation_gemv: bad sizes");
  if (B == 0 || N == 0) return FLUXB_OK;
  if (!vec || !w || !out) return set_error(FLUXB_ERR_BAD_ARG, "modulation_gemv: null pointer");
  if (K % 8 || !aligned16(w) || !aligned16(vec))
    return set_error(FLUXB_ERR_BAD_ARG, "modulation_gemv: K must be a multiple of 8 and pointers 16-byte aligned");
  if (K > 12288) return set_error(FLUXB_ERR_UNSUPPORTED, "modulation_gemv: K %lld > 12288", (long long)K);
  if (N > (int64_t)1 << 30) return set_error(FLUXB_ERR_UNSUPPORTED, "modulation_gemv: N %lld > 2^30", (long long)N);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(vec);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
  // Two blocks fit on an SM.  The grid is the number of row groups (one row per warp) divided
  // evenly over the fewest rounds that fit that many resident blocks: every warp then walks the
  // same number of rows (18432 rows, 16 warps per block: 288 blocks of 4 rounds, not 296 of 3.9).
  const int threads = light ? 128 : 512;
  const int64_t want = (N + threads / 32 - 1) / (threads / 32);
  const int64_t cap = (int64_t)sm_count() * 2;
  const int64_t rounds = (want + cap - 1) / cap;
  const unsigned grid = (unsigned)((want + rounds - 1) / rounds);
  const bool chunked = K % 1536 == 0;
  int64_t b0 = 0;
#define FLUXB_GEMV_LAUNCH(BT)                                                                          \
  {                                                                                                    \
    auto kern = chunked ? mod_gemv_mma_kernel<((BT) > 2 ? 2 : (BT))> : mod_gemv_kernel<BT>;            \
    const size_t smem = (size_t)(BT) * K * (chunked ? sizeof(__nv_bfloat16) : sizeof(float));          \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess)                                                                              \
      return set_error(FLUXB_ERR_CUDA, "modulation_gemv: cannot set shared memory size: %s",           \
                       cudaGetErrorString(e));                                                         \
    kern<<<grid, threads, smem, st>>>(vp, wp, bp, op, N, (int)K, b0, apply_silu, out_stride);          \
    b0 += (BT);                                                                                        \
  }
  while (b0 < B) {
    const int64_t left = B - b0;
    if (left >= 4 && !chunked) FLUXB_GEMV_LAUNCH(4)  // the mma form keeps 8 accumulators per batch row
    else if (left >= 2) FLUXB_GEMV_LAUNCH(2)
    else FLUXB_GEMV_LAUNCH(1)
  }
#undef FLUXB_GEMV_LAUNCH
  return launch_status("modulation_gemv");
}

extern "C" int fluxb_modulation_gemv(const void* vec, const void* w, const void* bias, void* out,
                                     int64_t B, int64_t N, int64_t K, int apply_silu,
                                     fluxb_stream_t stream) {
  return modulation_gemv_impl(vec, w, bias, out, B, N, K, N, apply_silu, false, stream);
}

extern "C" int fluxb_modulation_gemv_rows(const void* vec, const void* w, const void* bias, void* out,
                                          int64_t B, int64_t N, int64_t K, int64_t out_stride,
                                          int apply_silu, int light, fluxb_stream_t stream) {
  return modulation_gemv_impl(vec, w, bias, out, B, N, K, out_stride, apply_silu, light != 0, stream);
}
