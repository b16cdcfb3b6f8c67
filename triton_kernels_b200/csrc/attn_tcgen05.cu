// Non-causal flash attention forward for head_dim 128 or 64, bf16, on tcgen05 + TMEM.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles and walks the keys in
// tiles of 128.  Roles (384 threads = three warpgroups):
//   warps 0-3   softmax group 0: thread r owns query row r of tile 0
//   warps 4-7   softmax group 1: same for tile 1
//   warp  8     TMA producer: Q once, then K_j, V_j through a 4-slot ring of 32 KB tiles
//   warp  9     MMA issuer (whole warp walks the loop, one elected lane issues): S_t = Q_t K_j^T and
//               O_t += P_t V_j
//   warps 10-11 idle: they complete the third warpgroup, which hands most of its registers to the
//               softmax warpgroups (setmaxnreg: 56 against 224 per thread), so that a thread's 128
//               scores stay in registers without spills
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each.  P_t (bf16) is written back
// over the first 64 columns of S_t by the softmax threads and fed to the second MMA straight
// from TMEM, so probabilities never touch shared memory.  While group 0 does softmax on S_0 the
// tensor core works on tile 1 and vice versa.
// Softmax is the usual online form in base 2 with lazy rescaling: the running maximum used for
// the exponent only moves when a row maximum exceeds it by more than 8 (factor 256), which
// makes reading and rewriting O in TMEM rare.  Key tails are masked with -inf, query tails are
// not stored.  Every barrier wait is bounded.
#include "common.cuh"

namespace fluxb {
namespace attn {

// kD (kernel template parameter): head_dim, 64 or 128.
constexpr int BQ = 128;             // rows per query tile
constexpr int BKV = 128;            // keys per tile
constexpr int HALF_BYTES = 128 * 128;  // [128 rows][64 bf16] swizzled block
__host__ __device__ constexpr int tile_bytes(int d) { return (d / 64) * HALF_BYTES; }  // one Q, K or V tile: 128 rows x d
constexpr int KV_SLOTS = 4;
constexpr int THREADS = 384;
constexpr int TMEM_COLS = 512;
__host__ __device__ constexpr int smem_bytes(int d) { return 2 * tile_bytes(d) + KV_SLOTS * tile_bytes(d) + 1024 + 256; }
constexpr float kRescaleThreshold = 8.0f;
// kPolyEvery (kernel template parameter): every n-th pair of a row takes the polynomial exp2; 1000 = none.

struct Params {
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_sl;
  int Lq, Lk;
  float scale_log2;
  uint32_t v_lbo, v_sbo;
  DeviceStatus* status;
  // Scatter form (rows_per_rank > 0): query row r belongs to rank r / rows_per_rank and is
  // stored at o_rank[that rank] + batch*o_sb + head*o_sh + (r % rows_per_rank)*o_sl; the bases
  // may be other GPUs' memory (plain stores only).
  int rows_per_rank;
  __nv_bfloat16* o_rank[8];
  // Key-split form (k_splits > 1): CTA blockIdx.x handles query block blockIdx.x / k_splits and
  // the key tiles of split blockIdx.x % k_splits; it writes its normalised partial output as fp32
  // to part_o[split][batch][head][row][D] and the row's log2-sum-exp to part_lse[split][batch][head][row];
  // merge_splits_kernel combines the splits and stores the final rows (plain or scatter form).
  int k_splits;
  float* part_o;
  float* part_lse;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// exp2 of two values on the FMA pipes (no MUFU): round to the nearest integer n with the
// magic-number trick, evaluate a cubic for 2^f on f = x - n in [-0.5, 0.5] (max relative error
// 7.7e-5, far below the bf16 rounding of P), then add n into the exponent field.  Inputs are
// clamped at -126 so the exponent cannot wrap.  A share of every row goes this way so that the
// 16-lane-per-clock MUFU is not the only engine producing exponentials.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float kMagic = 12582912.0f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -126.0f);
  x.y = fmaxf(x.y, -126.0f);
  const float2 t = __fadd2_rn(x, make_float2(kMagic, kMagic));
  const float2 r = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
  const float2 f = __fadd2_rn(x, make_float2(-r.x, -r.y));
  float2 p = __ffma2_rn(f, make_float2(0.05508877709507942f, 0.05508877709507942f),
                        make_float2(0.242604061961174f, 0.242604061961174f));
  p = __ffma2_rn(p, f, make_float2(0.6932762265205383f, 0.6932762265205383f));
  p = __ffma2_rn(p, f, make_float2(0.9999289512634277f, 0.9999289512634277f));
  float2 out;
  out.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23));
  out.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23));
  return out;
}

// MMA issue with the accumulate flag known at compile time and descriptors given as
// (low word, high word): only the low word changes from one K step to the next.
template <int kAccumulate>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                       uint32_t b_hi, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(kAccumulate)
      : "memory");
}
template <int kAccumulate>
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                       uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(kAccumulate)
      : "memory");
}

template <int kPolyEvery, int kD>
__global__ void __launch_bounds__(THREADS, 1)
attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
            const __grid_constant__ CUtensorMap tm_v, const Params p) {
  constexpr int D = kD;
  constexpr int TILE_BYTES = tile_bytes(kD);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + 2 * TILE_BYTES;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(kv_smem + KV_SLOTS * TILE_BYTES);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + KV_SLOTS;
  uint64_t* s_full = kv_empty + KV_SLOTS;  // [2]
  uint64_t* p_full = s_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split = p.k_splits > 1 ? (int)(blockIdx.x % p.k_splits) : 0;
  const int q0 = (p.k_splits > 1 ? (int)(blockIdx.x / p.k_splits) : (int)blockIdx.x) * (2 * BQ);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int n_kv_all = (p.Lk + BKV - 1) / BKV;
  const int per_split = (n_kv_all + p.k_splits - 1) / p.k_splits;
  const int j_first = split * per_split;  // first key tile of this CTA (0 without a split)
  const int n_kv = min(n_kv_all - j_first, per_split);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);  // one arrival per softmax warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Registers move from the third warpgroup to the softmax warpgroups.  Each setmaxnreg sits
  // inside the branch whose code it governs, and what the one side releases (128 x 112) is
  // exactly what the other side takes (256 x 56): an increase waits for registers released
  // inside this CTA.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(q_smem + t * TILE_BYTES + hf * HALF_BYTES, &tm_q, q_full, hf * 64, q0 + t * BQ,
                      head, batch);
      bool ok = true;
      for (int i = 0; ok && i < 2 * n_kv; ++i) {  // i even: K_{i/2}, i odd: V_{i/2}
        const int slot = i % KV_SLOTS;
        const uint32_t phase = (i / KV_SLOTS) & 1;
        if (!mbar_wait(&kv_empty[slot], phase ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
        uint8_t* dst = kv_smem + slot * TILE_BYTES;
        mbar_expect_tx(&kv_full[slot], TILE_BYTES);
        const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
        const int row0 = (j_first + (i >> 1)) * BKV;
        for (int hf = 0; hf < D / 64; ++hf)
          tma_load_4d(dst + hf * HALF_BYTES, tm, &kv_full[slot], hf * 64, row0, head, batch);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (waits, address arithmetic) and one elected lane issues each
    // MMA and commit: control flow and descriptor words stay warp-uniform, which keeps the
    // per-instruction overhead of the issuing thread well below the 64 cycles an MMA lasts.
    {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, 0, 0);  // A = Q (K-major), B = K (K-major)
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, D, 0, 1);    // A = P (TMEM), B = V (MN-major)
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      bool ok = true;

      // Descriptor words.  High word: stride offset, descriptor version, 128-byte swizzle.
      const uint32_t hi_kmajor = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t hi_v = (p.v_sbo >> 4) | (1u << 14) | (2u << 29);
      const uint32_t v_lbo_field = ((p.v_lbo >> 4) & 0x3fffu) << 16;
      const uint32_t q_lo = (q_addr & 0x3ffffu) >> 4;
      const uint32_t kv_lo = (kv_addr & 0x3ffffu) >> 4;

      auto wait = [&](uint64_t* bar, uint32_t parity, int where) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.status, where)) != 0;
      };
      auto commit = [&](uint64_t* bar) {
        if (elect_one()) umma_commit(bar);
      };
      auto issue_qk = [&](int t, int slot) {
        const uint32_t qa = q_lo + t * (TILE_BYTES >> 4);
        const uint32_t ka = kv_lo + slot * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + t * 128;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            // 16 elements of head_dim per step: 32 bytes inside a 128-byte row, second half-block
            // after four steps
            const uint32_t off = (ks >> 2) * (HALF_BYTES >> 4) + (ks & 3) * 2;
            if (ks == 0) mma_ss<0>(d, qa + off, hi_kmajor, ka + off, hi_kmajor, idesc_qk);
            else mma_ss<1>(d, qa + off, hi_kmajor, ka + off, hi_kmajor, idesc_qk);
          }
        }
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint32_t va = (kv_lo + slot * (TILE_BYTES >> 4)) | v_lbo_field;
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t pa = tmem_base + t * 128;
        // 16 keys per step: 16 rows of 128 bytes in each half-block; 8 TMEM columns of P.
        if (elect_one()) {
          if (accumulate) mma_ts<1>(d, pa, va, hi_v, idesc_pv);
          else mma_ts<0>(d, pa, va, hi_v, idesc_pv);
#pragma unroll
          for (int ks = 1; ks < BKV / 16; ++ks) mma_ts<1>(d, pa + ks * 8, va + ks * 128, hi_v, idesc_pv);
        }
      };

      ok = wait(q_full, 0, 21);
      if (ok) ok = wait(&kv_full[0], 0, 22);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0, 0);
        commit(&s_full[0]);
        issue_qk(1, 0);
        commit(&s_full[1]);
        commit(&kv_empty[0]);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int iv = 2 * j + 1;
        const int v_slot = iv % KV_SLOTS;
        if (!wait(&kv_full[v_slot], (iv / KV_SLOTS) & 1, 23)) { ok = false; break; }
        const int ik = 2 * j + 2;
        const int k_slot = ik % KV_SLOTS;
        // The next K tile is waited for here, while this warp would be idle anyway until the
        // probabilities arrive, not between P.V and Q.K^T where the wait would sit on the chain
        // scores -> probabilities -> P.V -> next scores of a query tile.  (Its slot was freed an
        // iteration ago, so the load does not depend on anything issued below.)  K and V come
        // through TMA, the same proxy the MMAs read with: the barrier orders them by itself.
        if (j + 1 < n_kv && !wait(&kv_full[k_slot], (ik / KV_SLOTS) & 1, 25)) { ok = false; break; }
        for (int t = 0; t < 2; ++t) {
          if (!wait(&p_full[t], j & 1, 24)) { ok = false; break; }
          tc_fence_after_sync();
          issue_pv(t, v_slot, j > 0);
          if (t == 1) commit(&kv_empty[v_slot]);
          if (j + 1 < n_kv) {
            issue_qk(t, k_slot);
            commit(&s_full[t]);
            if (t == 1) commit(&kv_empty[k_slot]);
          } else {
            commit(&s_full[t]);  // final O_t complete
          }
        }
      }
    }
    __syncwarp();
  }
  } else {
    // ------------------------------------------------------------------ softmax groups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int t = warp >> 2;   // query tile / group
    const int quad = warp & 3;  // TMEM lane quadrant
    const int row = q0 + t * BQ + quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t s_addr = lane_base + t * 128;
    const uint32_t o_addr = lane_base + 256 + t * 128;
    float m_used = 0.f;  // running maximum (already multiplied by scale_log2) used in the exponent
    float l = 0.f;       // running sum of exp2
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, abort_flag, p.status, 31)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_wait_ld();

      const int valid = p.Lk - (j_first + j) * BKV;  // keys of this tile that exist
      if (valid < BKV) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= valid) s[i] = 0xff800000u;  // -inf
      }
      // four independent running maxima, two new elements per 3-input max
      float mxs[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) mxs[i] = __uint_as_float(s[i]);
#pragma unroll
      for (int i = 4; i < 128; i += 2)
        mxs[(i >> 1) & 3] = max3(mxs[(i >> 1) & 3], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
      const float mx_scaled = mx * p.scale_log2;

      if (j == 0) {
        m_used = mx_scaled;
      } else if (__any_sync(0xffffffffu, mx_scaled > m_used + kRescaleThreshold)) {
        // Move the exponent base for this warp's 32 rows and rescale their O rows in TMEM.  The
        // barrier just passed also covers the previous P·V of this tile, so O is quiescent.
        const float m_new = fmaxf(m_used, mx_scaled);
        const float alpha = ex2(m_used - m_new);
        l *= alpha;
        m_used = m_new;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_x32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(o_addr + c * 32, o);
        }
      }

      const float2 neg_m2 = make_float2(-m_used, -m_used);
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      float2 sums[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(
              make_float2(__uint_as_float(s[c * 32 + 2 * i]), __uint_as_float(s[c * 32 + 2 * i + 1])), scale2, neg_m2);
          float2 e;
          if ((i % kPolyEvery) == kPolyEvery - 1) {
            e = exp2_poly2(x);
          } else {
            e.x = ex2(x.x);
            e.y = ex2(x.y);
          }
          sums[i & 1] = __fadd2_rn(sums[i & 1], e);
          pk[i] = pack_bf16(e.x, e.y);
        }
        tmem_st_x16(s_addr + c * 16, pk);
      }
      l += (sums[0].x + sums[0].y) + (sums[1].x + sums[1].y);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);  // 4 arrivals per tile instead of 128 serialised ones
    }

    if (ok && mbar_wait(&s_full[t], n_kv & 1, abort_flag, p.status, 32)) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      if (p.k_splits > 1) {
        // partial result of this key range: normalised fp32 row + log2 of its sum of exponentials
        const int64_t prow = ((static_cast<int64_t>(split) * gridDim.z + batch) * gridDim.y + head) * p.Lq + row;
        if (row < p.Lq) p.part_lse[prow] = m_used + log2f(l);
        float* prow_o = p.part_o + prow * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_x32(o_addr + c * 32, o);
          tmem_wait_ld();
          if (row < p.Lq) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              *reinterpret_cast<float4*>(prow_o + c * 32 + g * 4) =
                  make_float4(__uint_as_float(o[g * 4 + 0]) * inv, __uint_as_float(o[g * 4 + 1]) * inv,
                              __uint_as_float(o[g * 4 + 2]) * inv, __uint_as_float(o[g * 4 + 3]) * inv);
          }
        }
      } else {
      __nv_bfloat16* orow = p.o + batch * p.o_sb + head * p.o_sh + (int64_t)row * p.o_sl;
      if (p.rows_per_rank > 0 && row < p.Lq) {
        const int owner = row / p.rows_per_rank;
        orow = p.o_rank[owner] + batch * p.o_sb + head * p.o_sh + (int64_t)(row - owner * p.rows_per_rank) * p.o_sl;
      }
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(o_addr + c * 32, o);
        tmem_wait_ld();
        if (row < p.Lq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
          }
        }
      }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Combines the partial results of a key-split launch: for every (batch, head, row) the splits'
// rows are weighted with exp2(lse_s - max lse) and normalised, then stored like the attention
// kernel stores its rows (plain or scatter form).  One warp per (batch, head, row); a lane owns
// D/32 consecutive output columns.
template <int kD>
__global__ void __launch_bounds__(256)
merge_splits_kernel(const Params p, int B, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t items = static_cast<int64_t>(B) * H * p.Lq;
  if (item >= items) return;
  const int row = static_cast<int>(item % p.Lq);
  const int head = static_cast<int>((item / p.Lq) % H);
  const int batch = static_cast<int>(item / (static_cast<int64_t>(p.Lq) * H));
  constexpr int PER = kD / 32;
  float mx = -INFINITY;
  for (int s_ = 0; s_ < p.k_splits; ++s_) mx = fmaxf(mx, p.part_lse[s_ * items + item]);
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  float wsum = 0.f;
  for (int s_ = 0; s_ < p.k_splits; ++s_) {
    const float w = exp2f(p.part_lse[s_ * items + item] - mx);
    wsum += w;
    const float* src = p.part_o + (s_ * items + item) * kD + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] += w * src[i];
  }
  const float inv = 1.0f / wsum;
  __nv_bfloat16* orow = p.o + batch * p.o_sb + head * p.o_sh + static_cast<int64_t>(row) * p.o_sl;
  if (p.rows_per_rank > 0) {
    const int owner = row / p.rows_per_rank;
    orow = p.o_rank[owner] + batch * p.o_sb + head * p.o_sh + static_cast<int64_t>(row - owner * p.rows_per_rank) * p.o_sl;
  }
  if (PER == 4) {
    uint2 w;
    w.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    w.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<uint2*>(orow + lane * 4) = w;
  } else {
    *reinterpret_cast<uint32_t*>(orow + lane * 2) = pack_bf16(acc[0] * inv, acc[1] * inv);
  }
}

}  // namespace attn
}  // namespace fluxb

using namespace fluxb;

static int encode_qkv_map(CUtensorMap* tm, const void* base, int64_t B, int64_t H, int64_t L, int64_t D,
                          int64_t sb, int64_t sh, int64_t sl) {
  // A size-1 dimension may come with any stride; give the encoder a harmless valid one.
  if (H == 1 || sh == 0) sh = sl * L;
  if (B == 1 || sb == 0) sb = sh * H;
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)L, (uint64_t)H, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)sl * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tmap_bf16(tm, base, 4, dims, strides, box);
}

static int attention_impl(const void* q, const void* k, const void* v, void* o, int64_t B,
                          int64_t H, int64_t Lq, int64_t Lk, int64_t D, int64_t q_sb,
                          int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                          int64_t v_sb, int64_t v_sh, int64_t v_sl, int64_t o_sb, int64_t o_sh,
                          int64_t o_sl, float sm_scale, void* const* o_bases, int n_ranks,
                          int64_t rows_per_rank, fluxb_stream_t stream, int k_splits = 1,
                          float* part_o = nullptr, float* part_lse = nullptr) {
  using namespace fluxb::attn;
  if (n_ranks > 0) {
    if (n_ranks > 8 || !o_bases || rows_per_rank <= 0 || rows_per_rank * n_ranks < Lq || rows_per_rank > (1 << 30))
      return set_error(FLUXB_ERR_BAD_ARG, "attention_scatter: need 1..8 output bases whose rows_per_rank rows cover Lq");
    for (int i = 0; i < n_ranks; ++i)
      if (!o_bases[i] || (reinterpret_cast<uintptr_t>(o_bases[i]) & 15))
        return set_error(FLUXB_ERR_BAD_ARG, "attention_scatter: output base %d is null or misaligned", i);
    o = o_bases[0];
  }
  if (D != 128 && D != 64)
    return set_error(FLUXB_ERR_UNSUPPORTED, "attention: head_dim %lld (64 and 128 are built)", (long long)D);
  if (B < 0 || H < 0 || Lq < 0 || Lk < 0) return set_error(FLUXB_ERR_BAD_ARG, "attention: negative size");
  if (B == 0 || H == 0 || Lq == 0) return FLUXB_OK;
  if (Lk == 0) return set_error(FLUXB_ERR_BAD_ARG, "attention: no keys");
  if (!q || !k || !v || !o) return set_error(FLUXB_ERR_BAD_ARG, "attention: null pointer");
  if (H > 65535 || B > 65535 || Lq > (1 << 30) || Lk > (1 << 30))
    return set_error(FLUXB_ERR_UNSUPPORTED, "attention: dimension too large");
  const int64_t strides[] = {q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, v_sb, v_sh, v_sl, o_sb, o_sh, o_sl};
  for (int64_t s : strides)
    if (s % 8 || s < 0) return set_error(FLUXB_ERR_BAD_ARG, "attention: strides must be non-negative multiples of 8 elements");
  if (q_sl < D || k_sl < D || v_sl < D || o_sl < D)
    return set_error(FLUXB_ERR_BAD_ARG, "attention: row stride below head_dim");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return set_error(FLUXB_ERR_BAD_ARG, "attention: pointers must be 16-byte aligned");

  CUtensorMap tm_q, tm_k, tm_v;
  int rc = encode_qkv_map(&tm_q, q, B, H, Lq, D, q_sb, q_sh, q_sl);
  if (rc == FLUXB_OK) rc = encode_qkv_map(&tm_k, k, B, H, Lk, D, k_sb, k_sh, k_sl);
  if (rc == FLUXB_OK) rc = encode_qkv_map(&tm_v, v, B, H, Lk, D, v_sb, v_sh, v_sl);
  if (rc != FLUXB_OK) return rc;

  Params p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.o_sb = o_sb; p.o_sh = o_sh; p.o_sl = o_sl;
  p.Lq = (int)Lq; p.Lk = (int)Lk;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  // V is consumed as the MN-major operand: 8-key groups are 1024 bytes apart (stride offset)
  // and the two 64-wide halves of head_dim are 16384 bytes apart (leading offset).
  p.v_lbo = HALF_BYTES;
  p.v_sbo = 1024;
  p.status = device_status_ptr();
  if (k_splits < 1 || k_splits > 8) return set_error(FLUXB_ERR_BAD_ARG, "attention: 1..8 key splits");
  if (k_splits > 1) {
    if (!part_o || !part_lse || (reinterpret_cast<uintptr_t>(part_o) & 15))
      return set_error(FLUXB_ERR_BAD_ARG, "attention: key splits need fp32 scratch for the partial rows and their log-sum-exp");
    const int64_t tiles = (Lk + BKV - 1) / BKV, per = (tiles + k_splits - 1) / k_splits;
    if ((k_splits - 1) * per >= tiles)
      return set_error(FLUXB_ERR_BAD_ARG, "attention: %d key splits leave one without key tiles (%lld tiles)", k_splits,
                       (long long)tiles);
    if (((Lq + 2 * BQ - 1) / (2 * BQ)) * k_splits > (1ll << 30))
      return set_error(FLUXB_ERR_UNSUPPORTED, "attention: dimension too large");
  }
  p.k_splits = k_splits;
  p.part_o = part_o;
  p.part_lse = part_lse;
  p.rows_per_rank = n_ranks > 0 ? (int)rows_per_rank : 0;
  for (int i = 0; i < 8; ++i) p.o_rank[i] = i < n_ranks ? static_cast<__nv_bfloat16*>(o_bases[i]) : nullptr;

  // Every fourth pair of a row takes the polynomial exp2.
  auto kern = D == 128 ? attn_kernel<4, 128> : attn_kernel<4, 64>;
  const int smem = smem_bytes((int)D);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "attention: cannot set shared memory size: %s", cudaGetErrorString(e));
  dim3 grid((unsigned)(((Lq + 2 * BQ - 1) / (2 * BQ)) * k_splits), (unsigned)H, (unsigned)B);
  kern<<<grid, THREADS, smem, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, p);
  if (k_splits > 1) {
    const int64_t items = B * H * Lq;
    auto merge = D == 128 ? merge_splits_kernel<128> : merge_splits_kernel<64>;
    merge<<<(unsigned)((items + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, (int)B, (int)H);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "attention: launch failed: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

extern "C" int fluxb_attention(const void* q, const void* k, const void* v, void* o, int64_t B,
                               int64_t H, int64_t Lq, int64_t Lk, int64_t D, int64_t q_sb,
                               int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                               int64_t v_sb, int64_t v_sh, int64_t v_sl, int64_t o_sb, int64_t o_sh,
                               int64_t o_sl, float sm_scale, fluxb_stream_t stream) {
  return attention_impl(q, k, v, o, B, H, Lq, Lk, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, v_sb, v_sh, v_sl, o_sb,
                        o_sh, o_sl, sm_scale, nullptr, 0, 0, stream);
}

extern "C" int fluxb_attention_scatter(const void* q, const void* k, const void* v, void* const* o_bases,
                                       int n_ranks, int64_t rows_per_rank, int64_t B, int64_t H, int64_t Lq,
                                       int64_t Lk, int64_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl,
                                       int64_t k_sb, int64_t k_sh, int64_t k_sl, int64_t v_sb, int64_t v_sh,
                                       int64_t v_sl, int64_t o_sb, int64_t o_sh, int64_t o_sl, float sm_scale,
                                       fluxb_stream_t stream) {
  if (n_ranks <= 0) return set_error(FLUXB_ERR_BAD_ARG, "attention_scatter: no output bases");
  return attention_impl(q, k, v, nullptr, B, H, Lq, Lk, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, v_sb, v_sh, v_sl,
                        o_sb, o_sh, o_sl, sm_scale, o_bases, n_ranks, rows_per_rank, stream);
}

extern "C" int fluxb_attention_split(const void* q, const void* k, const void* v, void* o, void* const* o_bases,
                                     int n_ranks, int64_t rows_per_rank, int64_t B, int64_t H, int64_t Lq,
                                     int64_t Lk, int64_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb,
                                     int64_t k_sh, int64_t k_sl, int64_t v_sb, int64_t v_sh, int64_t v_sl,
                                     int64_t o_sb, int64_t o_sh, int64_t o_sl, float sm_scale, int k_splits,
                                     float* part_o, float* part_lse, fluxb_stream_t stream) {
  if (n_ranks < 0) return set_error(FLUXB_ERR_BAD_ARG, "attention_split: negative rank count");
  return attention_impl(q, k, v, n_ranks > 0 ? nullptr : o, B, H, Lq, Lk, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, v_sb,
                        v_sh, v_sl, o_sb, o_sh, o_sl, sm_scale, n_ranks > 0 ? o_bases : nullptr, n_ranks, rows_per_rank,
                        stream, k_splits, part_o, part_lse);
}
