// y = x · w^T with fused epilogues, as persistent, warp-specialised tcgen05 kernels.
//
// Both kernels have one TMA producer warp (streams 64-wide K slices of x and w, bf16, 128-byte
// swizzle, through a shared-memory ring), one MMA warp (the whole warp walks the loop, an elected
// lane issues tcgen05.mma from shared memory into one of two 256-column fp32 accumulators in
// TMEM; tcgen05.commit releases ring slots and publishes finished accumulators) and epilogue
// warps that read their 32-lane TMEM quadrant with tcgen05.ld and apply bias / GELU /
// gate+residual in fp32.  Two accumulators let the epilogue of tile i overlap the main loop of
// tile i+1.
//
//   gemm_pair_kernel (default, 320 threads)  clusters of two CTAs share a 256x256 tile through
//               cta_group::2 MMAs; 5-stage ring of 32 KB per CTA; EIGHT epilogue warps in two
//               groups that take alternate 64-column pieces of a tile, each group with its own
//               swizzled staging tile, named barrier and TMA-store-issuing thread; up to four
//               problems per launch.  Second instantiation: the q|k|v head epilogue (QK RMS norm,
//               RoPE, head-major layout through a 5-D TMA store).
//   gemm_kernel (FLUXB_GEMM_PAIR=0, 192 threads)  one CTA per 128x256 tile, 4-stage ring of
//               48 KB, four epilogue warps, direct 16-byte stores.
//
// Tiles are handed out statically (tile = id + i * stride) in an L2-aware order (tile_coords).
// Edge tiles rely on TMA zero fill for loads and on TMA clipping / masks for stores.  Every
// barrier wait is bounded.
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

namespace fluxb {

namespace gemm {
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct Params {
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  __nv_bfloat16* y2;
  const __nv_bfloat16* resid;
  const __nv_bfloat16* gate;
  int64_t ldy, ldy2, ldr, gate_stride, rows_per_batch;
  int M, N, K;
  int split, epi, epi2, round_before_act;
  int tiles_m, tiles_n, num_tiles;
  int pair_stages;  // CTA-pair kernel: ring depth in use (<= gemm2::STAGES)
  int raster_band_n, raster_group;  // tile order, see tile_coords
  DeviceStatus* status;
  // EPI_QKV_HEADS (CTA-pair kernel only): the N = 3*heads*128 columns are q | k | v of `heads`
  // heads; q and k rows are RMS-normalised per head with qk_scale[0/1] (if given) and rotated
  // with pe (if given), and everything is stored head-major through the 5-D map in tm_y.
  const float* pe;                     // [l_total, 64, 2, 2]
  const __nv_bfloat16* qk_scale[2];    // [128] each
  int row_offset, heads, l_total;      // joint position of this problem's first token
  float eps;
  // Scatter form of EPI_QKV_HEADS (scat_groups > 0): head h of q goes to
  // scat_base[h / scat_hpg] + b*scat_sb + (h % scat_hpg)*scat_sh + l*scat_sl, k and v scat_koff /
  // scat_voff elements further; the bases may be other GPUs' memory (plain 16-byte stores only).
  __nv_bfloat16* scat_base[8];
  int scat_groups, scat_hpg;
  int64_t scat_sb, scat_sh, scat_sl, scat_koff, scat_voff;
};
constexpr int EPI_QKV_HEADS = 3;  // internal epilogue code, set by fluxb_linear_qkv_grouped

// Tile order.  The tiles running at one time form a gm x gn rectangle of the output; all of
// them walk K in step, so each x row-block and w row-block is fetched from HBM once per
// rectangle and served from L2 to the others.  Across rectangles one operand is kept and the
// other swept:
//   band_n == 0: groups of `group` row-blocks of x are kept while all column-blocks are swept
//   band_n == 1: bands of `group` column-blocks (rows of w) are kept while x is swept
__device__ __forceinline__ void tile_coords(const Params& p, int tile, int tiles_m, int& m_blk, int& n_blk) {
  if (p.raster_band_n == 0) {
    const int per_group = p.raster_group * p.tiles_n;
    const int group = tile / per_group;
    const int first_m = group * p.raster_group;
    const int gsize = min(tiles_m - first_m, p.raster_group);
    const int in_group = tile - group * per_group;
    m_blk = first_m + in_group % gsize;
    n_blk = in_group / gsize;
  } else {
    const int per_band = p.raster_group * tiles_m;
    const int band = tile / per_band;
    const int first_n = band * p.raster_group;
    const int bsize = min(p.tiles_n - first_n, p.raster_group);
    const int in_band = tile - band * per_band;
    n_blk = first_n + in_band % bsize;
    m_blk = in_band / bsize;
  }
}

// Applies the epilogue to 32 consecutive columns of one output row held in registers.
// With `stage_row` == nullptr the 8-column pieces go straight to global memory with 16-byte
// stores.  Otherwise they go to this row's 128-byte line of a shared-memory staging tile in the
// 128-byte-swizzle layout (16-byte piece q of row r sits at ((q ^ (r & 7)) * 16), from where a
// TMA store writes full lines; `piece0` is the index of the first piece within the line.
__device__ __forceinline__ void epilogue_chunk(const Params& p, const uint32_t (&acc)[32], int row,
                                               int col0, bool second, uint8_t* stage_row = nullptr,
                                               int piece0 = 0, int swz = 0) {
  const int epi = second ? p.epi2 : p.epi;
  __nv_bfloat16* out = second ? p.y2 : p.y;
  const int64_t ld = second ? p.ldy2 : p.ldy;
  const int out_col0 = second ? col0 - p.split : col0;
  const bool row_ok = row < p.M;
  const int64_t b = (epi == FLUXB_EPI_GATE_RESID && row_ok) ? row / p.rows_per_batch : 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int col = col0 + j * 8;
    if (col >= p.N) break;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(acc[j * 8 + e]);
    if (p.bias != nullptr) {
      const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
      v[0] += bf16_lo(bv.x); v[1] += bf16_hi(bv.x); v[2] += bf16_lo(bv.y); v[3] += bf16_hi(bv.y);
      v[4] += bf16_lo(bv.z); v[5] += bf16_hi(bv.z); v[6] += bf16_lo(bv.w); v[7] += bf16_hi(bv.w);
    }
    if (epi == FLUXB_EPI_GELU) {
      if (p.round_before_act) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(__float2bfloat16_rn(v[e]));
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
    } else if (epi == FLUXB_EPI_GATE_RESID) {
      if (row_ok) {
        const uint4 rv = *reinterpret_cast<const uint4*>(p.resid + (int64_t)row * p.ldr + col);
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(p.gate + b * p.gate_stride + col));
        v[0] = bf16_lo(rv.x) + bf16_lo(gv.x) * v[0]; v[1] = bf16_hi(rv.x) + bf16_hi(gv.x) * v[1];
        v[2] = bf16_lo(rv.y) + bf16_lo(gv.y) * v[2]; v[3] = bf16_hi(rv.y) + bf16_hi(gv.y) * v[3];
        v[4] = bf16_lo(rv.z) + bf16_lo(gv.z) * v[4]; v[5] = bf16_hi(rv.z) + bf16_hi(gv.z) * v[5];
        v[6] = bf16_lo(rv.w) + bf16_lo(gv.w) * v[6]; v[7] = bf16_hi(rv.w) + bf16_hi(gv.w) * v[7];
      }
    }
    uint4 o;
    o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]);
    o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
    if (stage_row != nullptr) {
      *reinterpret_cast<uint4*>(stage_row + (((piece0 + j) ^ swz) << 4)) = o;  // rows/cols past the edge are clipped by the TMA store
    } else if (row_ok) {
      *reinterpret_cast<uint4*>(out + (int64_t)row * ld + out_col0 + j * 8) = o;
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(p, tile, p.tiles_m, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(a_dst, &tm_a, &full_bar[stage], kb * BK, m_blk * BM);
          tma_load_2d(b_dst, &tm_b, &full_bar[stage], kb * BK, n_blk * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp walks the loop and an elected lane issues (warp-uniform descriptors).
    {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 2))) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3))) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t adesc = make_smem_desc(a_addr, 16, 1024);
          const uint64_t bdesc = make_smem_desc(a_addr + A_BYTES, 16, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              // 16 bf16 along K = 32 bytes = 2 descriptor address units
              umma_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) umma_commit(&acc_full[acc]);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++local) {
      int m_blk, n_blk;
      tile_coords(p, tile, p.tiles_m, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m_blk * BM + quad * 32 + lane;
      const int n0 = n_blk * BN;
      const bool second = n0 >= p.split;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (n0 + c * 32 >= p.N) break;  // uniform
        uint32_t r[32];
        tmem_ld_x32(t_addr + c * 32, r);
        tmem_wait_ld();
        epilogue_chunk(p, r, row, n0 + c * 32, second);
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm

// ----------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster share one 256x256 output tile.  Each CTA loads its
// own 128 rows of x and only HALF of the w tile (128 rows); one thread of the even ("leader")
// CTA issues cta_group::2 MMAs (M=256, N=256, K=16) that run on both SMs, each tensor core
// reading the other half of w from its partner's shared memory.  Per SM this halves the
// shared-memory and L2 traffic for w, which is what bounds the single-CTA kernel.
//   - both CTAs' TMA loads count on the leader's "full" barrier (pair form of the bulk copy)
//   - slot release and accumulator-full are tcgen05.commit arrivals delivered to the barrier
//     at the same offset in BOTH CTAs, so each CTA's producer / epilogue waits locally
//   - accumulator-empty is counted on the leader (4 epilogue warps x 2 CTAs, remote arrive)
// (Relaying the slot release through the leader's producer with a remote mbarrier arrive
// instead was measured at half the throughput.)
// ----------------------------------------------------------------------------------------
namespace gemm2 {
using gemm::Params;
using gemm::epilogue_chunk;
using gemm::tile_coords;
constexpr int BM = 128;       // rows of x per CTA (256 per pair)
constexpr int BN = 256;       // output columns per tile
constexpr int BNH = 128;      // rows of w loaded by each CTA
constexpr int BK = 64;
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OUT_CHUNK_COLS = 64;                       // output columns per staged TMA store
constexpr int OUT_BUF_BYTES = BM * OUT_CHUNK_COLS * 2;   // 128 rows x 128 bytes
constexpr int THREADS = 320;  // TMA warp, MMA warp, two groups of four epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BUF_BYTES + 1024 + 256;
constexpr int MAX_PROBLEMS = 4;

// Up to four GEMMs that differ in operands, outputs and row counts run as ONE persistent
// launch: their tiles are concatenated (problem 0's tiles first) and dealt round-robin to the
// CTA pairs.  A small problem (the 512-token text stream) would fill a third of the machine on
// its own; riding along with the image stream's GEMM it fills the tail of that launch instead.
struct Problem {
  CUtensorMap tm_a, tm_b;
  CUtensorMap tm_y, tm_y2;  // outputs (columns below / from `split`), box 64 columns x 128 rows
  Params p;
  int tile_start;  // index of this problem's first tile in the concatenated order
  int tiles_m;     // 256-row blocks
};
struct Grouped {
  Problem prob[MAX_PROBLEMS];
  int count;
  int total_tiles;
  int pair_stages;
};

static_assert(sizeof(Grouped) <= 4096, "kernel parameters are limited to 4 KB");

__device__ __forceinline__ int find_problem(const Grouped& g, int tile) {
  int i = 0;
#pragma unroll
  for (int k = 1; k < MAX_PROBLEMS; ++k)
    if (k < g.count && tile >= g.prob[k].tile_start) i = k;
  return i;
}

// Epilogue of one 128-row x 256-column tile (two heads of q, of k or of v) for EPI_QKV_HEADS:
// bias, rounding to bf16 (the projection's output precision in the reference), per-head RMS norm
// and rotation for q and k in fp32 with one rounding at the end, head-major 5-D TMA stores at
// (d, l, head, batch, part).  One thread of each epilogue group owns one row.  The row's sums of
// squares are taken in a first sweep over the accumulator (by both groups); in the second sweep
// a thread works 16 columns at a time for BOTH heads, because the rotation entries depend on
// the row and the pair only: each batch of eight pe entries is loaded once and used for the
// two heads.  The two groups take alternate 16-column steps; staging tile hh collects head hh
// from both groups and is stored by group hh's issuing thread.
__device__ __forceinline__ void qkv_load16(const Params& p, uint32_t taddr, int col, float (&x)[16]) {
  uint32_t r[16];
  tmem_ld_x16(taddr, r);
  tmem_wait_ld();
#pragma unroll
  for (int e = 0; e < 16; ++e) x[e] = __uint_as_float(r[e]);
  if (p.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col + j * 8));
      x[j * 8 + 0] += bf16_lo(bv.x); x[j * 8 + 1] += bf16_hi(bv.x); x[j * 8 + 2] += bf16_lo(bv.y); x[j * 8 + 3] += bf16_hi(bv.y);
      x[j * 8 + 4] += bf16_lo(bv.z); x[j * 8 + 5] += bf16_hi(bv.z); x[j * 8 + 6] += bf16_lo(bv.w); x[j * 8 + 7] += bf16_hi(bv.w);
    }
  }
#pragma unroll
  for (int e = 0; e < 16; ++e) x[e] = __bfloat162float(__float2bfloat16_rn(x[e]));
}

template <bool kScatter>
__device__ __forceinline__ void qkv_tile_epilogue(const Params& p, const CUtensorMap* tm, uint32_t t_addr, int part,
                                                  int head0, int n0, int heads_in_tile, int b, int l0, int r_local,
                                                  bool rows_ok, uint8_t* out_stage, int eg, bool store_issuer,
                                                  int rows_left) {
  const __nv_bfloat16* w = part < 2 ? p.qk_scale[part] : nullptr;
  const bool rotate = part < 2 && p.pe != nullptr && rows_ok && (!kScatter || r_local < rows_left);
  float rstd0 = 1.f, rstd1 = 1.f;
  if (w != nullptr) {
#pragma unroll 1
    for (int hh = 0; hh < heads_in_tile; ++hh) {
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < 128; c += 16) {
        float x[16];
        qkv_load16(p, t_addr + hh * 128 + c, n0 + hh * 128 + c, x);
#pragma unroll
        for (int e = 0; e < 16; ++e) ss += x[e] * x[e];
      }
      const float r = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
      if (hh == 0) rstd0 = r; else rstd1 = r;
    }
  }
  const float4* pr = reinterpret_cast<const float4*>(p.pe) + static_cast<int64_t>(l0 + r_local) * 64;
  // This group's four steps of 16 columns: steps eg and eg + 2 of each 64-column piece.  The pe
  // entries of the next step are requested before the current one is worked on.
  float4 f_next[8];
  if (rotate) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f_next[i] = __ldg(pr + (eg * 16) / 2 + i);
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = it >> 1;
    const int step = eg + 2 * (it & 1);
    const int c = piece * 64 + step * 16;  // column within the head
    if ((it & 1) == 0) {
      // both staging tiles must have been read out by the stores of the piece before (each
      // issuer waits for its own), and nobody writes before both issuers are through
      if (store_issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      asm volatile("bar.sync 3, 256;" ::: "memory");
    }
    float4 f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f_next[i];
    if (rotate && it < 3) {
      const int cn = ((it + 1) >> 1) * 64 + (eg + 2 * ((it + 1) & 1)) * 16;
#pragma unroll
      for (int i = 0; i < 8; ++i) f_next[i] = __ldg(pr + cn / 2 + i);
    }
#pragma unroll 1
    for (int hh = 0; hh < heads_in_tile; ++hh) {
      float x[16];
      qkv_load16(p, t_addr + hh * 128 + c, n0 + hh * 128 + c, x);
      if (w != nullptr) {
        const float r = hh == 0 ? rstd0 : rstd1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + c + j * 8));
          x[j * 8 + 0] *= r * bf16_lo(wv.x); x[j * 8 + 1] *= r * bf16_hi(wv.x);
          x[j * 8 + 2] *= r * bf16_lo(wv.y); x[j * 8 + 3] *= r * bf16_hi(wv.y);
          x[j * 8 + 4] *= r * bf16_lo(wv.z); x[j * 8 + 5] *= r * bf16_hi(wv.z);
          x[j * 8 + 6] *= r * bf16_lo(wv.w); x[j * 8 + 7] *= r * bf16_hi(wv.w);
        }
      }
      if (rotate) {
        // pe[l, i] = {f00, f01, f10, f11}: out[2i] = f00 x[2i] + f01 x[2i+1], out[2i+1] = f10 x[2i] + f11 x[2i+1]
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float a0 = x[2 * i], a1 = x[2 * i + 1];
          x[2 * i] = f[i].x * a0 + f[i].y * a1;
          x[2 * i + 1] = f[i].z * a0 + f[i].w * a1;
        }
      }
      uint8_t* line = out_stage + hh * OUT_BUF_BYTES + r_local * 128;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const float* v = &x[jj * 8];
        uint4 o;
        o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]);
        o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
        *reinterpret_cast<uint4*>(line + (((step * 2 + jj) ^ (r_local & 7)) << 4)) = o;
      }
    }
    if ((it & 1) == 1) {
      fence_proxy_async_smem();
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (kScatter) {
        // All 256 epilogue threads copy the finished staging tiles out with plain 16-byte stores:
        // eight consecutive threads write one row's 128 bytes of one head.  The destination of a
        // head depends on its group (another GPU's arena under sequence parallelism), and rows
        // beyond the stream's end are skipped one by one, so stream lengths need not be
        // multiples of 128 here.  The barrier at the top of the next piece orders these reads
        // before the tiles are written again.
        const int tid = eg * 128 + r_local;
        const int64_t part_off = part == 0 ? 0 : (part == 1 ? p.scat_koff : p.scat_voff);
#pragma unroll 1
        for (int hh = 0; hh < heads_in_tile; ++hh) {
          const int head = head0 + hh;
          const int grp = head / p.scat_hpg;
          __nv_bfloat16* dst_head = p.scat_base[grp] + part_off + b * p.scat_sb + (head - grp * p.scat_hpg) * p.scat_sh +
                                    piece * 64;
          const uint8_t* src_tile = out_stage + hh * OUT_BUF_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int idx = tid + 256 * k;
            const int r = idx >> 3, q = idx & 7;
            if (r < rows_left) {
              const uint4 v = *reinterpret_cast<const uint4*>(src_tile + r * 128 + ((q ^ (r & 7)) << 4));
              *reinterpret_cast<uint4*>(dst_head + (int64_t)(l0 + r) * p.scat_sl + q * 8) = v;
            }
          }
        }
      } else
      // group eg's issuer stores staging tile eg = head eg of the tile
      if (store_issuer && rows_ok && eg < heads_in_tile) {
        asm volatile(
            "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                reinterpret_cast<uint64_t>(tm)),
            "r"(smem_u32(out_stage + eg * OUT_BUF_BYTES)), "r"(piece * 64), "r"(l0), "r"(head0 + eg), "r"(b), "r"(part)
            : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
  }
}

// kMode selects the epilogue at compile time, so that the ordinary kernel carries none of the other
// forms' code or register pressure:
//   0  ordinary (bias / GELU / gate+residual / column split)
//   1  q|k|v columns through the head epilogue, columns from `split` on ordinary
template <int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ Grouped g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* out_stage = smem + STAGES * STAGE_BYTES;  // two 16 KB output staging tiles
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(out_stage + 2 * OUT_BUF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = g.total_tiles;
  DeviceStatus* const status = g.prob[0].p.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 16);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < g.count; ++i) {
      tma_prefetch_desc(&g.prob[i].tm_a);
      tma_prefetch_desc(&g.prob[i].tm_b);
      tma_prefetch_desc(&g.prob[i].tm_y);
      tma_prefetch_desc(&g.prob[i].tm_y2);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // partner's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        const Problem& pr = g.prob[find_problem(g, tile)];
        const Params& p = pr.p;
        const int num_kb = (p.K + BK - 1) / BK;
        int m_blk, n_blk;
        tile_coords(p, tile - pr.tile_start, pr.tiles_m, m_blk, n_blk);
        const int row0 = m_blk * 2 * BM + (int)rank * BM;
        const int col0 = n_blk * BN + (int)rank * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1, abort_flag, status, 41)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t full_addr = map_to_cta(smem_u32(&full_bar[stage]), 0);
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          tma_load_2d_pair(a_dst, &pr.tm_a, full_addr, kb * BK, row0);
          tma_load_2d_pair(a_dst + A_BYTES, &pr.tm_b, full_addr, kb * BK, col0);
          if (++stage == g.pair_stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp of the leader CTA walks the loop and an elected lane issues, so that
    // addresses and descriptors stay warp-uniform.
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs, ++local) {
        const int num_kb = (g.prob[find_problem(g, tile)].p.K + BK - 1) / BK;
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait_cluster(&acc_empty[acc], acc_phase ^ 1, abort_flag, status, 43))) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait_cluster(&full_bar[stage], phase, abort_flag, status, 44))) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t adesc = make_smem_desc(a_addr, 16, 1024);
          const uint64_t bdesc = make_smem_desc(a_addr + A_BYTES, 16, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit_pair_both(&empty_bar[stage]);
          }
          if (++stage == g.pair_stages) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) umma_commit_pair_both(&acc_full[acc]);
      }
    }
    __syncwarp();
  } else {
    // Two groups of four epilogue warps (warps 2-5 and 6-9; warp w reads TMEM lane quadrant w % 4).
    // A tile leaves in four 64-column pieces; group eg takes pieces eg and eg + 2 with a staging
    // tile, a named barrier and a store-issuing thread of its own.  One warp per scheduler was
    // not enough to cover the latencies inside a piece (accumulator load, bias / gate / residual
    // loads, GELU): measured per tile and CTA, 20 000 cycles for the plain epilogue, 28 000 with
    // GELU and 37 000 with gate + residual, against a main loop of 24 600 cycles at K = 3072.
    const int quad = warp & 3;
    const int eg = (warp - 2) >> 2;
    const int bar_id = 1 + eg;
    int local = 0;
    bool ok = true;
    const uint32_t acc_empty_leader0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    const bool store_issuer = warp == 2 + 4 * eg && lane == 0;
    for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs, ++local) {
      const Problem& pr = g.prob[find_problem(g, tile)];
      const Params& p = pr.p;
      int m_blk, n_blk;
      tile_coords(p, tile - pr.tile_start, pr.tiles_m, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row0 = m_blk * 2 * BM + (int)rank * BM;
      const int r_local = quad * 32 + lane;
      const int row = row0 + r_local;
      const int n0 = n_blk * BN;
      const bool second = n0 >= p.split;
      if (!mbar_wait_cluster(&acc_full[acc], acc_phase, abort_flag, status, 45)) { ok = false; break; }
      tc_fence_after_sync();
      const CUtensorMap* tm_out = second ? &pr.tm_y2 : &pr.tm_y;
      const int out_col0 = second ? n0 - p.split : n0;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      // The tile leaves in four 64-column pieces: registers -> swizzled staging tile in shared
      // memory -> one TMA store of full 128-byte lines.  (Storing 16 bytes per thread straight
      // to global memory, 32 different rows per warp instruction, cost 9 % of the GEMM.)
      if (kMode >= 1 && !second) {
        const int hd = p.heads * 128;
        const int part = n0 / hd;
        const int head0 = (n0 - part * hd) / 128;
        const bool rows_ok = row0 < p.M;  // M is a multiple of 128 here: a CTA's rows exist or do not
        const int b = row0 / (int)p.rows_per_batch;
        const int l0 = p.row_offset + (row0 - b * (int)p.rows_per_batch);
        const int heads_in_tile = (p.split - n0) >= BN ? BN / 128 : (p.split - n0) / 128;  // split = 3*heads*128
        qkv_tile_epilogue<kMode == 2>(p, &pr.tm_y, t_addr, part, head0, n0, heads_in_tile, b, l0, r_local, rows_ok,
                                      out_stage, eg, store_issuer, p.M - row0);
      } else {
      // ordinary columns: this group's two pieces, through its own staging tile
      uint8_t* buf = out_stage + eg * OUT_BUF_BYTES;
      uint8_t* line = buf + r_local * 128;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = eg + 2 * i;
        if (n0 + c * OUT_CHUNK_COLS < p.N) {  // uniform
          uint32_t r0[32], r1[32];
          tmem_ld_x32(t_addr + c * OUT_CHUNK_COLS, r0);
          tmem_ld_x32(t_addr + c * OUT_CHUNK_COLS + 32, r1);
          tmem_wait_ld();
          // this group's previous store must have read the staging tile out
          if (store_issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          epilogue_chunk(p, r0, row, n0 + c * OUT_CHUNK_COLS, second, line, 0, r_local & 7);
          epilogue_chunk(p, r1, row, n0 + c * OUT_CHUNK_COLS + 32, second, line, 4, r_local & 7);
          fence_proxy_async_smem();
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          if (store_issuer) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(tm_out)),
                         "r"(smem_u32(buf)), "r"(out_col0 + c * OUT_CHUNK_COLS), "r"(row0)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + acc * 8);
    }
    if (store_issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // staging tiles outlive their stores
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its partner may still touch its memory
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace fluxb

using namespace fluxb;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static bool use_pair_kernel() {
  // CTA pairs (256x256 tiles) unless FLUXB_GEMM_PAIR=0 asks for the single-CTA kernel.
  static const int pair_env = [] {
    const char* s = getenv("FLUXB_GEMM_PAIR");
    return (s != nullptr && *s != 0) ? atoi(s) : 1;
  }();
  return pair_env != 0;
}

// Validates one problem, encodes its tensor maps and fills its kernel parameters.
static int prepare_problem(const fluxb_linear_problem& a, int64_t N, int64_t K, int epi, int64_t split, int epi2,
                           int round_before_act, bool use_pair, CUtensorMap* tm_a, CUtensorMap* tm_b,
                           fluxb::gemm::Params* out) {
  using namespace fluxb::gemm;
  const int64_t M = a.M;
  if (M <= 0 || N <= 0 || K <= 0) return set_error(FLUXB_ERR_BAD_ARG, "linear: bad sizes");
  if (M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2)
    return set_error(FLUXB_ERR_UNSUPPORTED, "linear: dimension too large");
  if (!a.x || !a.w || !a.y) return set_error(FLUXB_ERR_BAD_ARG, "linear: null pointer");
  if (split < 0 || split > N) return set_error(FLUXB_ERR_BAD_ARG, "linear: split outside [0, N]");
  if (split < N) {
    if (!a.y2) return set_error(FLUXB_ERR_BAD_ARG, "linear: split < N needs a second output");
    if (split % BN) return set_error(FLUXB_ERR_BAD_ARG, "linear: split must be a multiple of %d", BN);
    if (a.ldy2 % 8 || !aligned16(a.y2)) return set_error(FLUXB_ERR_BAD_ARG, "linear: second output misaligned");
  }
  if (K % 8 || a.ldx % 8 || a.ldw % 8 || N % 8 || a.ldy % 8 || a.ldx < K || a.ldw < K)
    return set_error(FLUXB_ERR_BAD_ARG, "linear: K, N and row strides must be multiples of 8 (and strides >= K)");
  if (!aligned16(a.x) || !aligned16(a.w) || !aligned16(a.y) || !aligned16(a.bias))
    return set_error(FLUXB_ERR_BAD_ARG, "linear: pointers must be 16-byte aligned");
  const int epis[2] = {epi, split < N ? epi2 : FLUXB_EPI_NONE};
  for (int e : epis) {
    if (e != FLUXB_EPI_NONE && e != FLUXB_EPI_GELU && e != FLUXB_EPI_GATE_RESID)
      return set_error(FLUXB_ERR_UNSUPPORTED, "linear: unknown epilogue %d", e);
    if (e == FLUXB_EPI_GATE_RESID) {
      if (!a.resid || !a.gate || a.rows_per_batch <= 0 || a.ldr % 8 || a.gate_stride % 8 || !aligned16(a.resid) ||
          !aligned16(a.gate))
        return set_error(FLUXB_ERR_BAD_ARG, "linear: gate/residual epilogue needs aligned resid, gate and rows_per_batch > 0");
    }
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)a.ldx * 2};
    const uint32_t box[2] = {BK, BM};
    int rc = encode_tmap_bf16(tm_a, a.x, 2, dims, strides, box);
    if (rc != FLUXB_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)a.ldw * 2};
    const uint32_t box[2] = {BK, (uint32_t)(use_pair ? fluxb::gemm2::BNH : BN)};
    int rc = encode_tmap_bf16(tm_b, a.w, 2, dims, strides, box);
    if (rc != FLUXB_OK) return rc;
  }
  Params& p = *out;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.y = static_cast<__nv_bfloat16*>(a.y);
  p.y2 = static_cast<__nv_bfloat16*>(a.y2);
  p.resid = static_cast<const __nv_bfloat16*>(a.resid);
  p.gate = static_cast<const __nv_bfloat16*>(a.gate);
  p.ldy = a.ldy; p.ldy2 = a.ldy2; p.ldr = a.ldr; p.gate_stride = a.gate_stride;
  p.rows_per_batch = a.rows_per_batch > 0 ? a.rows_per_batch : 1;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.split = (int)split; p.epi = epi; p.epi2 = epi2; p.round_before_act = round_before_act;
  p.tiles_m = (int)((M + BM - 1) / BM);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.status = device_status_ptr();
  p.pe = nullptr; p.qk_scale[0] = p.qk_scale[1] = nullptr; p.row_offset = 0; p.heads = 0; p.l_total = 0; p.eps = 0.f;
  p.scat_groups = 0; p.scat_hpg = 1; p.scat_sb = p.scat_sh = p.scat_sl = p.scat_koff = p.scat_voff = 0;
  for (int gi = 0; gi < 8; ++gi) p.scat_base[gi] = nullptr;
  p.pair_stages = fluxb::gemm2::STAGES;
  {
    // Keep the smaller operand resident in L2 when it fits, sweep the larger one.
    const int row_blk = use_pair ? 256 : 128;
    const int tm = (int)((M + row_blk - 1) / row_blk);
    const int tn = p.tiles_n;
    const int concurrent = use_pair ? sm_count() / 2 : sm_count();
    const double a_bytes = 2.0 * (double)M * (double)K, w_bytes = 2.0 * (double)N * (double)K;
    const double keep_limit = 48e6;
    if (a_bytes <= w_bytes) {
      p.raster_band_n = 0;  // keep x row-blocks
      p.raster_group = a_bytes <= keep_limit ? tm : (concurrent / tn > 1 ? concurrent / tn : 1);
    } else {
      p.raster_band_n = 1;  // keep w row-blocks
      p.raster_group = w_bytes <= keep_limit ? tn : (concurrent / tm > 1 ? concurrent / tm : 1);
    }
    if (p.raster_group < 1) p.raster_group = 1;
  }
  return FLUXB_OK;
}

extern "C" int fluxb_linear_grouped(const fluxb_linear_problem* problems, int count, int64_t N, int64_t K, int epi,
                                    int64_t split, int epi2, int round_before_act, fluxb_stream_t stream) {
  using namespace fluxb::gemm;
  if (count < 0 || (count > 0 && problems == nullptr)) return set_error(FLUXB_ERR_BAD_ARG, "linear_grouped: bad problem list");
  if (count > fluxb::gemm2::MAX_PROBLEMS)
    return set_error(FLUXB_ERR_UNSUPPORTED, "linear_grouped: at most %d problems per launch", fluxb::gemm2::MAX_PROBLEMS);
  if (N < 0 || K <= 0) return set_error(FLUXB_ERR_BAD_ARG, "linear: bad sizes");
  const bool use_pair = use_pair_kernel();
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  fluxb::gemm2::Grouped g;
  g.count = 0;
  g.total_tiles = 0;
  g.pair_stages = fluxb::gemm2::STAGES;
  for (int i = 0; i < count; ++i) {
    if (problems[i].M < 0) return set_error(FLUXB_ERR_BAD_ARG, "linear: negative M");
    if (problems[i].M == 0 || N == 0) continue;  // nothing to compute for this one
    fluxb::gemm2::Problem& pr = g.prob[g.count];
    int rc = prepare_problem(problems[i], N, K, epi, split, epi2, round_before_act, use_pair, &pr.tm_a, &pr.tm_b, &pr.p);
    if (rc != FLUXB_OK) return rc;
    if (!use_pair) {  // single-CTA kernel: one launch per problem
      cudaError_t e = cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "linear: cannot set shared memory size: %s", cudaGetErrorString(e));
      const int grid = pr.p.num_tiles < sm_count() ? pr.p.num_tiles : sm_count();
      gemm_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(pr.tm_a, pr.tm_b, pr.p);
      continue;
    }
    {
      const fluxb_linear_problem& a = problems[i];
      const int64_t n_first = split < N ? split : N;
      const uint32_t box[2] = {fluxb::gemm2::OUT_CHUNK_COLS, fluxb::gemm2::BM};
      const uint64_t dims[2] = {(uint64_t)n_first, (uint64_t)a.M};
      const uint64_t strides[1] = {(uint64_t)a.ldy * 2};
      rc = n_first > 0 ? encode_tmap_bf16(&pr.tm_y, a.y, 2, dims, strides, box) : FLUXB_OK;
      if (rc != FLUXB_OK) return rc;
      if (split < N) {
        const uint64_t dims2[2] = {(uint64_t)(N - split), (uint64_t)a.M};
        const uint64_t strides2[1] = {(uint64_t)a.ldy2 * 2};
        rc = encode_tmap_bf16(&pr.tm_y2, a.y2, 2, dims2, strides2, box);
        if (rc != FLUXB_OK) return rc;
        if (n_first == 0) pr.tm_y = pr.tm_y2;
      } else {
        pr.tm_y2 = pr.tm_y;
      }
    }
    pr.tiles_m = (int)((problems[i].M + 255) / 256);
    pr.tile_start = g.total_tiles;
    g.total_tiles += pr.tiles_m * pr.p.tiles_n;
    ++g.count;
  }
  if (use_pair && g.count > 0) {
    auto kern = fluxb::gemm2::gemm_pair_kernel<0>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fluxb::gemm2::SMEM_BYTES);
    if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "linear: cannot set shared memory size: %s", cudaGetErrorString(e));
    const int pairs = g.total_tiles < sm_count() / 2 ? g.total_tiles : sm_count() / 2;
    kern<<<2 * pairs, fluxb::gemm2::THREADS, fluxb::gemm2::SMEM_BYTES, st>>>(g);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "linear: launch failed: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

struct QkvScatter {  // destination of the scatter form, see fluxb_linear_qkv_grouped_scatter
  void* const* bases;
  int n_groups;
  int64_t k_off, v_off, sb, sh, sl;
};

static int linear_qkv_grouped_impl(const fluxb_linear_problem* problems, const fluxb_qkv_stream* streams,
                                   int count, int64_t B, int64_t H, int64_t D, int64_t L_total, int64_t K,
                                   void* qkv_out, const QkvScatter* scat, float eps, int64_t N2, int epi2,
                                   int round_before_act, fluxb_stream_t stream) {
  using namespace fluxb::gemm;
  if (count < 1 || count > fluxb::gemm2::MAX_PROBLEMS || !problems || !streams)
    return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: 1..%d problems with their stream descriptions", fluxb::gemm2::MAX_PROBLEMS);
  if (!use_pair_kernel()) return set_error(FLUXB_ERR_UNSUPPORTED, "linear_qkv_grouped: needs the CTA-pair kernel (FLUXB_GEMM_PAIR=0 is set)");
  if (D != 128) return set_error(FLUXB_ERR_UNSUPPORTED, "linear_qkv_grouped: head_dim %lld (only 128)", (long long)D);
  // A 256-column tile holds two heads and is normalised as a whole with q's, k's or no scale: the
  // q|k and k|v boundaries (multiples of H*D) must therefore fall on tile boundaries.
  if ((H * D) % 256)
    return set_error(FLUXB_ERR_UNSUPPORTED, "linear_qkv_grouped: %lld heads (the head count must be even)", (long long)H);
  if (B <= 0 || H <= 0 || L_total <= 0 || K <= 0 || B > 65535 || H > 65535 || L_total > (1 << 30))
    return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: bad sizes");
  if (scat == nullptr) {
    if (!qkv_out || !aligned16(qkv_out)) return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: output null or misaligned");
  } else {
    if (scat->n_groups < 1 || scat->n_groups > 8 || !scat->bases || H % scat->n_groups)
      return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped_scatter: 1..8 head groups that divide the head count");
    for (int i = 0; i < scat->n_groups; ++i)
      if (!scat->bases[i] || !aligned16(scat->bases[i]))
        return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped_scatter: output base %d is null or misaligned", i);
    if (scat->k_off % 8 || scat->v_off % 8 || scat->sb % 8 || scat->sh % 8 || scat->sl % 8 || scat->sl < D)
      return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped_scatter: offsets and strides must be multiples of 8 elements");
  }
  if (N2 < 0 || N2 % 8) return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: N2 must be a non-negative multiple of 8");
  if (epi2 != FLUXB_EPI_NONE && epi2 != FLUXB_EPI_GELU)
    return set_error(FLUXB_ERR_UNSUPPORTED, "linear_qkv_grouped: the extra columns take no epilogue or GELU");
  const int64_t N_qkv = 3 * H * D;
  const int64_t N = N_qkv + N2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  fluxb::gemm2::Grouped g;
  g.count = 0;
  g.total_tiles = 0;
  g.pair_stages = fluxb::gemm2::STAGES;
  // one 5-D map over [3, B, H, L_total, D] for all problems
  CUtensorMap tm_out;
  if (scat == nullptr) {
    const uint64_t dims[5] = {(uint64_t)D, (uint64_t)L_total, (uint64_t)H, (uint64_t)B, 3};
    const uint64_t strides[4] = {(uint64_t)D * 2, (uint64_t)L_total * D * 2, (uint64_t)H * L_total * D * 2,
                                 (uint64_t)B * H * L_total * D * 2};
    const uint32_t box[5] = {fluxb::gemm2::OUT_CHUNK_COLS, fluxb::gemm2::BM, 1, 1, 1};
    int rc = encode_tmap_bf16(&tm_out, qkv_out, 5, dims, strides, box);
    if (rc != FLUXB_OK) return rc;
  }
  for (int i = 0; i < count; ++i) {
    fluxb_linear_problem a = problems[i];
    const fluxb_qkv_stream& sdesc = streams[i];
    const int64_t Ls = a.rows_per_batch;
    // The head-major form leaves through 128-row TMA boxes; the scatter form masks row by row, so
    // with one batch item any stream length and offset will do.
    const int64_t align = (scat != nullptr && B == 1) ? 1 : 128;
    if (a.M <= 0 || Ls <= 0 || a.M != B * Ls || Ls % align)
      return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: each stream needs M = B * rows_per_batch with rows_per_batch a multiple of 128");
    if (sdesc.row_offset < 0 || sdesc.row_offset % align || sdesc.row_offset + Ls > L_total)
      return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: row_offset must be a multiple of 128 inside the joint sequence");
    if ((sdesc.q_scale == nullptr) != (sdesc.k_scale == nullptr) || !aligned16(sdesc.q_scale) || !aligned16(sdesc.k_scale) ||
        !aligned16(sdesc.pe))
      return set_error(FLUXB_ERR_BAD_ARG, "linear_qkv_grouped: scales go together; scales and pe must be 16-byte aligned");
    a.y = scat == nullptr ? qkv_out : scat->bases[0]; a.ldy = D;  // the q|k|v columns do not leave through y
    a.resid = nullptr; a.gate = nullptr;
    if (N2 == 0) a.y2 = nullptr;
    fluxb::gemm2::Problem& pr = g.prob[g.count];
    int rc = prepare_problem(a, N, K, FLUXB_EPI_NONE, N_qkv, epi2, round_before_act, true, &pr.tm_a, &pr.tm_b, &pr.p);
    if (rc != FLUXB_OK) return rc;
    pr.p.epi = EPI_QKV_HEADS;
    pr.p.rows_per_batch = Ls;
    pr.p.pe = sdesc.pe;
    pr.p.qk_scale[0] = static_cast<const __nv_bfloat16*>(sdesc.q_scale);
    pr.p.qk_scale[1] = static_cast<const __nv_bfloat16*>(sdesc.k_scale);
    pr.p.row_offset = (int)sdesc.row_offset;
    pr.p.heads = (int)H;
    pr.p.l_total = (int)L_total;
    pr.p.eps = eps;
    if (scat != nullptr) {
      pr.p.scat_groups = scat->n_groups;
      pr.p.scat_hpg = (int)(H / scat->n_groups);
      for (int gi = 0; gi < 8; ++gi) pr.p.scat_base[gi] = gi < scat->n_groups ? static_cast<__nv_bfloat16*>(scat->bases[gi]) : nullptr;
      pr.p.scat_sb = scat->sb; pr.p.scat_sh = scat->sh; pr.p.scat_sl = scat->sl;
      pr.p.scat_koff = scat->k_off; pr.p.scat_voff = scat->v_off;
      tm_out = pr.tm_a;  // never used for a store in this form; any valid map will do for the prefetch
    }
    pr.tm_y = tm_out;
    pr.tm_y2 = tm_out;
    if (N2 > 0) {  // extra columns [3*H*D, 3*H*D + N2): an ordinary output with epilogue epi2
      const uint32_t box[2] = {fluxb::gemm2::OUT_CHUNK_COLS, fluxb::gemm2::BM};
      const uint64_t dims2[2] = {(uint64_t)N2, (uint64_t)a.M};
      const uint64_t strides2[1] = {(uint64_t)a.ldy2 * 2};
      rc = encode_tmap_bf16(&pr.tm_y2, a.y2, 2, dims2, strides2, box);
      if (rc != FLUXB_OK) return rc;
    }
    pr.tiles_m = (int)((a.M + 255) / 256);
    pr.tile_start = g.total_tiles;
    g.total_tiles += pr.tiles_m * pr.p.tiles_n;
    ++g.count;
  }
  auto kern = scat == nullptr ? fluxb::gemm2::gemm_pair_kernel<1> : fluxb::gemm2::gemm_pair_kernel<2>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fluxb::gemm2::SMEM_BYTES);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "linear_qkv_grouped: cannot set shared memory size: %s", cudaGetErrorString(e));
  const int pairs = g.total_tiles < sm_count() / 2 ? g.total_tiles : sm_count() / 2;
  kern<<<2 * pairs, fluxb::gemm2::THREADS, fluxb::gemm2::SMEM_BYTES, st>>>(g);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "linear_qkv_grouped: launch failed: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

extern "C" int fluxb_linear_qkv_grouped(const fluxb_linear_problem* problems, const fluxb_qkv_stream* streams,
                                        int count, int64_t B, int64_t H, int64_t D, int64_t L_total, int64_t K,
                                        void* qkv_out, float eps, int64_t N2, int epi2, int round_before_act,
                                        fluxb_stream_t stream) {
  return linear_qkv_grouped_impl(problems, streams, count, B, H, D, L_total, K, qkv_out, nullptr, eps, N2, epi2,
                                 round_before_act, stream);
}

extern "C" int fluxb_linear_qkv_grouped_scatter(const fluxb_linear_problem* problems, const fluxb_qkv_stream* streams,
                                                int count, int64_t B, int64_t H, int64_t D, int64_t L_total,
                                                int64_t K, void* const* group_bases, int n_groups, int64_t k_off,
                                                int64_t v_off, int64_t o_sb, int64_t o_sh, int64_t o_sl, float eps,
                                                int64_t N2, int epi2, int round_before_act, fluxb_stream_t stream) {
  const QkvScatter scat{group_bases, n_groups, k_off, v_off, o_sb, o_sh, o_sl};
  return linear_qkv_grouped_impl(problems, streams, count, B, H, D, L_total, K, nullptr, &scat, eps, N2, epi2,
                                 round_before_act, stream);
}

extern "C" int fluxb_linear(const void* x, const void* w, const void* bias, void* y, int64_t M,
                            int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int epi,
                            void* y2, int64_t ldy2, int64_t split, int epi2, const void* resid,
                            int64_t ldr, const void* gate, int64_t gate_stride,
                            int64_t rows_per_batch, int round_before_act, fluxb_stream_t stream) {
  fluxb_linear_problem a;
  a.x = x; a.w = w; a.bias = bias; a.y = y; a.M = M; a.ldx = ldx; a.ldw = ldw; a.ldy = ldy;
  a.y2 = y2; a.ldy2 = ldy2; a.resid = resid; a.ldr = ldr; a.gate = gate; a.gate_stride = gate_stride;
  a.rows_per_batch = rows_per_batch;
  if (M < 0 || N < 0 || K <= 0) return set_error(FLUXB_ERR_BAD_ARG, "linear: bad sizes");
  return fluxb_linear_grouped(&a, 1, N, K, epi, split, epi2, round_before_act, stream);
}
