// TF32 GEMM on the 5th-generation tensor cores (sm_100a):
//   C[M,N] (+)= op(A) * op(B), row-major fp32 operands, fp32 accumulate in TMEM.
//
// Structure (persistent, warp-specialised, one CTA per SM):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into a
//               128-byte-swizzled shared-memory ring (STAGES deep)
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma.kind::tf32
//               (128 x BN x 8 per instruction) into one of two TMEM accumulators
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, store / accumulate
//               to global while the MMA warp already works on the next tile
// Transposed operands are handled by MN-major shared-memory descriptors, so no
// operand is ever transposed in memory.  Optional split-K writes partial sums to
// a workspace that a second, deterministic kernel reduces.
//
// Role in the reference: cublasSgemm / cublasSgemmStridedBatched
// (src/ops/MatrixMult.cu:4-72, src/ops/BatchMatrixMult.cu:4-43).
#include "tc_common.cuh"
#include "scratch.h"

#include <mutex>
#include <unordered_map>
#include <string>
#include <cstdio>
#include <cstring>
#include <cstdlib>

using namespace tsb;

namespace {

constexpr int BM = 128;
constexpr int BK = 32;                 // 32 tf32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;
constexpr int A_STAGE_BYTES = BM * BK * 4;

struct GemmParams {
  float* c;
  float* ws;          // split-K partials [splits][batch][M][N] (null when splits == 1)
  int m, n, k;
  int batch;
  long long ldc, sc;  // C row stride / batch stride (elements)
  int splits;
  int accumulate;
  int tiles_m, tiles_n;
  int kblocks;        // ceil(K / BK)
  int a_chunked, b_chunked;   // MN-major operand mapped (32 cols, k, chunk of 32 cols, batch): one box per stage
  int* status;
  // Head layout (attention): the batch is (outer, head) with `heads` heads, and an operand flagged here is stored
  // [outer][row][head][col] instead of [outer][head][row][col].  Its tensor map then has the head as batch
  // dimension and the rows of all outer batches in one row dimension; batch (o, h) starts `o * shift` rows in.
  int heads;                  // 0: plain batched GEMM
  int a_heads, b_heads, c_heads;
  int a_shift, b_shift;       // rows per outer batch of A / B in memory (M or K rows, N or K rows)
  long long sc2;              // C stride of the outer batch when c_heads (sc is then the head stride)
};

// Order in which the persistent CTAs walk the output tiles: groups of TILE_GROUP_M tile rows, column by column
// inside a group.  The CTAs that run at the same time (consecutive tile indices) then share TILE_GROUP_M row
// panels of A and a handful of column panels of B, which together stay in L2, instead of one or two rows of A
// and every panel of B.
constexpr int TILE_GROUP_M = 8;
__device__ __forceinline__ void tile_mn(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = TILE_GROUP_M * tiles_n;
  const int g = tile / per_group, r = tile - g * per_group;
  const int m_first = g * TILE_GROUP_M;
  const int rows = min(TILE_GROUP_M, tiles_m - m_first);
  tn = r / rows;
  tm = m_first + (r - tn * rows);
}

// Tensor-map batch coordinate and row offset of A and B, and the offset of C, for batch index b.
struct BatchAt {
  int ab, ar, bb, br;
  long long c_off;
};
__device__ __forceinline__ BatchAt batch_at(const GemmParams& p, int b) {
  BatchAt t;
  t.ab = t.bb = b; t.ar = t.br = 0;
  t.c_off = (long long)b * p.sc;
  if (p.heads > 0) {
    const int o = b / p.heads, h = b - o * p.heads;
    if (p.a_heads) { t.ab = h; t.ar = o * p.a_shift; }
    if (p.b_heads) { t.bb = h; t.br = o * p.b_shift; }
    if (p.c_heads) t.c_off = (long long)o * p.sc2 + (long long)h * p.sc;
  }
  return t;
}

template <int BN>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + C::STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.tiles_m * p.tiles_n;
  const long long items = (long long)tiles * p.batch * p.splits;
  const int kb_per_split = (p.kblocks + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int tile = (int)(item % tiles);
        const long long rest = item / tiles;
        const int b = (int)(rest % p.batch);
        const int split = (int)(rest / p.batch);
        int tm, tn;
        tile_mn(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kblocks, kb0 + kb_per_split);
        const BatchAt at = batch_at(p, b);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x101)) { ok = false; break; }
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          uint8_t* sa = smem_a + s * A_STAGE_BYTES;
          uint8_t* sb = smem_b + s * C::B_STAGE_BYTES;
          const int k0 = kb * BK;
          // (the row dimension in memory is M / N for a K-major operand and K for an MN-major one)
          if (!A_MN) {
            tma_load_3d(sa, &tmA, &full[s], k0, m0 + at.ar, at.ab);
          } else if (p.a_chunked) {
            tma_load_4d(sa, &tmA, &full[s], 0, k0 + at.ar, m0 >> 5, at.ab);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              tma_load_3d(sa + c * (BK * 128), &tmA, &full[s], m0 + c * 32, k0 + at.ar, at.ab);
          }
          if (!B_MN) {
            tma_load_3d(sb, &tmB, &full[s], k0, n0 + at.br, at.bb);
          } else if (p.b_chunked) {
            tma_load_4d(sb, &tmB, &full[s], 0, k0 + at.br, n0 >> 5, at.bb);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              tma_load_3d(sb + c * (BK * 128), &tmB, &full[s], n0 + c * 32, k0 + at.br, at.bb);
          }
        }
      }
      if (!ok) {   // let copies that are still in flight land before the CTA goes away
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // descriptor halves: K-major operands step 32 bytes per MMA inside the 128B swizzle row,
      // MN-major ones (32-byte-atom swizzle, chunks of 32 columns BK*128 bytes apart) 1024 bytes
      constexpr uint32_t A_HI = A_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t B_HI = B_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t A_KSTEP = (A_MN ? 1024 : UMMA_K * 4) >> 4, B_KSTEP = (B_MN ? 1024 : UMMA_K * 4) >> 4;
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), A_MN ? BK * 128 : 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), B_MN ? BK * 128 : 16);
      uint32_t it = 0, acc_it = 0;
      bool ok = true, ready = false;
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++acc_it) {
        const long long rest = item / tiles;
        const int split = (int)(rest / p.batch);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kblocks, kb0 + kb_per_split);
        const int acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, 0x102)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!ready && !mbar_wait(&full[s], ph, p.status, 0x103)) { ok = false; break; }
          {   // probe the next stage now; the answer arrives while this stage's MMAs are issued
            const uint32_t it2 = it + 1;
            ready = mbar_test(&full[it2 % C::STAGES], (it2 / C::STAGES) & 1);
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (C::B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_tf32(d_tmem, smem_desc_join(A_HI, a_lo + k * A_KSTEP), smem_desc_join(B_HI, b_lo + k * B_KSTEP),
                      idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);     // frees the smem stage when these MMAs retire
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;              // TMEM lane quarter this warp may access
    uint32_t acc_it = 0;
    bool ok = true;
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++acc_it) {
      const int tile = (int)(item % tiles);
      const long long rest = item / tiles;
      const int b = (int)(rest % p.batch);
      const int split = (int)(rest / p.batch);
      int tm, tn;
      tile_mn(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      const int kb0 = split * kb_per_split;
      const bool has_k = kb0 < p.kblocks;     // an empty K range contributes zeros
      if (!mbar_wait(&tfull[acc], acc_ph, p.status, 0x104)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      float* crow;
      bool accumulate;
      if (p.splits > 1) {
        crow = p.ws + ((long long)(split * p.batch + b) * p.m + row) * p.n;
        accumulate = false;
      } else {
        crow = p.c + batch_at(p, b).c_off + (long long)row * p.ldc;
        accumulate = p.accumulate != 0;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        if (has_k) {
          tmem_ld_32x32(tmem_base + acc * BN + ((uint32_t)(q * 32) << 16) + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        const int col = n0 + c0;
        if (row < p.m && col < p.n) {
          float* dst = crow + col;
          const bool vec_ok = (col + 32 <= p.n) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          if (vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dst + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dst + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.n) dst[j] = accumulate ? dst[j] + v[j] : v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): a cluster of two CTAs on an SM pair computes one 256 x 256 tile.
// Each CTA stages its own 128 rows of A and its own 128 columns of B (32 KB per k-block instead of
// 48 KB, so six stages fit and each byte of B crosses L2 -> SM once per pair); the leader's elected
// thread issues 256 x 256 x 8 MMAs that run on both SMs; each CTA drains its own 128 x 256
// accumulator half from its own TMEM.  Barriers:
//   full[s]   leader only: 1 arrival (its producer, with the byte count of BOTH CTAs' boxes)
//   empty[s]  per CTA: 1 arrival, by the multicast commit of the leader's MMAs
//   tfull[a]  per CTA: 1 arrival, multicast commit after the last k-block of a tile
//   tempty[a] leader only: 8 arrivals (four epilogue warps of each CTA)
// ---------------------------------------------------------------------------------------------
constexpr int P2_BN = 256;                               // tile columns of the pair
constexpr int P2_BNH = P2_BN / 2;                        // columns of B staged per CTA
constexpr int P2_B_STAGE_BYTES = P2_BNH * BK * 4;
constexpr int P2_STAGE_BYTES = A_STAGE_BYTES + P2_B_STAGE_BYTES;   // 32 KB
constexpr int P2_STAGES = 6;
constexpr int P2_SMEM_BYTES = P2_STAGES * P2_STAGE_BYTES + 1024 + 256;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + P2_STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P2_STAGES * P2_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + P2_STAGES;
  uint64_t* tfull = bars + 2 * P2_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const long long pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {                                    // the same warp in both CTAs, as the pair allocation requires
    tmem_alloc_2sm(tmem_slot, 512);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ptm = (p.m + 255) / 256, ptn = (p.n + P2_BN - 1) / P2_BN;
  const int tiles = ptm * ptn;
  const long long items = (long long)tiles * p.batch;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long item = pair; item < items && ok; item += npairs) {
        const int tile = (int)(item % tiles);
        const int b = (int)(item / tiles);
        int tm, tn;
        tile_mn(tile, ptm, ptn, tm, tn);
        const int m0 = tm * 256 + (int)rank * 128;           // this CTA's rows of A
        const int n0 = tn * P2_BN + (int)rank * P2_BNH;      // this CTA's columns of B
        const BatchAt at = batch_at(p, b);
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % P2_STAGES;
          const uint32_t ph = (it / P2_STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x111)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * P2_STAGE_BYTES);
          uint8_t* sa = smem_a + s * A_STAGE_BYTES;
          uint8_t* sb = smem_b + s * P2_B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!A_MN) tma_load_3d_2sm(sa, &tmA, &full[s], k0, m0 + at.ar, at.ab);
          else tma_load_4d_2sm(sa, &tmA, &full[s], 0, k0 + at.ar, m0 >> 5, at.ab);
          if (!B_MN) tma_load_3d_2sm(sb, &tmB, &full[s], k0, n0 + at.br, at.bb);
          else tma_load_4d_2sm(sb, &tmB, &full[s], 0, k0 + at.br, n0 >> 5, at.bb);
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(256, P2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_HI = A_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t B_HI = B_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t A_KSTEP = (A_MN ? 1024 : UMMA_K * 4) >> 4, B_KSTEP = (B_MN ? 1024 : UMMA_K * 4) >> 4;
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), A_MN ? BK * 128 : 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), B_MN ? BK * 128 : 16);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (long long item = pair; item < items && ok; item += npairs, ++acc_it) {
        const int acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, 0x112)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P2_BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % P2_STAGES;
          const uint32_t ph = (it / P2_STAGES) & 1;
          if (!mbar_wait(&full[s], ph, p.status, 0x113)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (P2_B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_tf32_2sm(d_tmem, smem_desc_join(A_HI, a_lo + k * A_KSTEP), smem_desc_join(B_HI, b_lo + k * B_KSTEP),
                          idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_2sm(&empty[s], 3);      // both CTAs may refill this stage once the MMAs retire
        }
        if (ok) umma_commit_2sm(&tfull[acc], 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own TMEM half)
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (long long item = pair; item < items && ok; item += npairs, ++acc_it) {
      const int tile = (int)(item % tiles);
      const int b = (int)(item / tiles);
      int tm, tn;
      tile_mn(tile, ptm, ptn, tm, tn);
      const int m0 = tm * 256 + (int)rank * 128;
      const int n0 = tn * P2_BN;
      const int acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, p.status, 0x114)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      float* crow = p.c + batch_at(p, b).c_off + (long long)row * p.ldc;
      const bool accumulate = p.accumulate != 0;
#pragma unroll 1
      for (int c0 = 0; c0 < P2_BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tmem_base + acc * P2_BN + ((uint32_t)(q * 32) << 16) + c0, v);
        tmem_ld_wait();
        const int col = n0 + c0;
        if (row < p.m && col < p.n) {
          float* dst = crow + col;
          const bool vec_ok = (col + 32 <= p.n) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          if (vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dst + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dst + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.n) dst[j] = accumulate ? dst[j] + v[j] : v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);   // the leader's MMA thread counts both CTAs' warps
    }
  }

  // Nobody leaves (and nobody frees TMEM) while the partner may still signal or read.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

// Deterministic split-K reduction: c (+)= sum_s ws[s]
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, float* __restrict__ c, int splits,
                                     long long per_split, int m, int n, long long ldc, long long sc,
                                     int accumulate) {
  const long long total = per_split;   // = batch * m * n
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[s * per_split + i];
    const long long b = i / ((long long)m * n);
    const long long r = (i / n) % m;
    const long long col = i % n;
    float* dst = c + b * sc + r * ldc + col;
    *dst = accumulate ? *dst + acc : acc;
  }
}

// Plain SIMT fallback for shapes the tensor-map rules exclude (leading dimension
// not a multiple of 4 floats, unaligned base).  Tiny problems only.
__global__ void gemm_simt_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                 int m, int n, int k, long long lda, long long ldb, long long ldc, int ta, int tb,
                                 long long sa, long long sb, long long sc, int accumulate) {
  __shared__ float as[16][17], bs[16][17];
  const int bz = blockIdx.z;
  a += bz * sa; b += bz * sb; c += bz * sc;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < k; k0 += 16) {
    const int ka = k0 + tx, kb = k0 + ty;
    as[ty][tx] = (row < m && ka < k) ? (ta ? a[(long long)ka * lda + row] : a[(long long)row * lda + ka]) : 0.f;
    bs[ty][tx] = (col < n && kb < k) ? (tb ? b[(long long)col * ldb + kb] : b[(long long)kb * ldb + col]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) acc += as[ty][kk] * bs[kk][tx];
    __syncthreads();
  }
  if (row < m && col < n) {
    float* dst = c + (long long)row * ldc + col;
    *dst = accumulate ? *dst + acc : acc;
  }
}

}  // namespace

// ---------------------------------------------------------------------------- host
namespace tsb_host {

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_b,
                  const uint32_t* box, bool atom32) {
  return make_tmap_f32_swz(out, base, rank, dims, strides_b, box, atom32 ? 1 : 0);
}

int make_tmap_f32_swz(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_b,
                      const uint32_t* box, int swizzle) {
  const int atom32 = swizzle;      // cache key field: the swizzle code
  EncodeTiledFn fn = encode_fn();
  if (!fn) return TSB_ERR_TMAP;
  // cache: identical descriptors are re-used across steps (addresses are stable under the pool)
  struct Key {
    const void* base; int rank; int atom32; uint64_t d[5], s[4]; uint32_t b[5];
    bool operator==(const Key& o) const { return std::memcmp(this, &o, sizeof(Key)) == 0; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
      size_t h = 1469598103934665603ull;
      for (size_t i = 0; i < sizeof(Key) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
      return h;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  Key key;
  std::memset(&key, 0, sizeof(key));
  key.base = base; key.rank = rank; key.atom32 = atom32;
  for (int i = 0; i < rank; ++i) { key.d[i] = dims[i]; key.b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.s[i] = strides_b[i];
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return TSB_OK; }
  }
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_b[i];
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                               : (swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return TSB_ERR_TMAP | ((int)r << 8);
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache[key] = *out;
  }
  return TSB_OK;
}

int make_tmap_im2col_f32(CUtensorMap* out, const void* base, int C, int W, int H, int N, const int* lower,
                         const int* upper, int channels, int pixels, int stride_w, int stride_h, bool atom32) {
  typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeIm2colFn fn = nullptr;
  static int driver_version = 0;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeIm2colFn>(p);
    cudaDriverGetVersion(&driver_version);
  });
  if (!fn) return TSB_ERR_TMAP;
  for (int i = 0; i < 2; ++i)
    if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return TSB_ERR_UNSUPPORTED;
  struct Key {
    const void* base; int v[13];
    bool operator==(const Key& o) const { return std::memcmp(this, &o, sizeof(Key)) == 0; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&k);
      size_t h = 1469598103934665603ull;
      for (size_t i = 0; i < sizeof(Key) / 4; ++i) h = (h ^ w[i]) * 1099511628211ull;
      return h;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  Key key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  const int vals[13] = {C, W, H, N, lower[0], lower[1], upper[0], upper[1], channels, pixels, stride_w, stride_h,
                        atom32 ? 1 : 0};
  std::memcpy(key.v, vals, sizeof(vals));
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return TSB_OK; }
  }
  cuuint64_t gd[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t gs[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
  cuuint32_t es[4] = {1, (cuuint32_t)stride_w, (cuuint32_t)stride_h, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gd, gs, lower, upper,
                  (cuuint32_t)channels, (cuuint32_t)pixels, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return TSB_ERR_TMAP | ((int)r << 8);
  // Drivers up to CUDA 13.1 encode im2col maps of tensors smaller than 128 KiB with a flag that
  // makes the load misbehave; CUTLASS clears it the same way
  // (cute/atom/copy_traits_sm90_im2col.hpp, make_im2col_tma_copy_desc).
  if (driver_version <= 13010 && (size_t)C * W * H * N * 4 < 131072)
    reinterpret_cast<uint64_t*>(out)[1] &= ~(1ull << 21);
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache[key] = *out;
  }
  return TSB_OK;
}

static int* g_status_host = nullptr;   // pinned, mapped: one word per device
static int* g_status_dev[64] = {nullptr};

int* status_word(cudaStream_t) {
  int dev = 0;
  cudaGetDevice(&dev);
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  if (!g_status_host) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), 64 * sizeof(int), cudaHostAllocMapped |
                      cudaHostAllocPortable) != cudaSuccess)
      return nullptr;
    std::memset(g_status_host, 0, 64 * sizeof(int));
  }
  if (!g_status_dev[dev]) {
    int* d = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), g_status_host, 0) != cudaSuccess) return nullptr;
    g_status_dev[dev] = d + dev;
  }
  return g_status_dev[dev];
}

int peek_status() {
  int dev = 0;
  cudaGetDevice(&dev);
  return g_status_host ? *(volatile int*)(g_status_host + dev) : 0;
}

int read_status(cudaStream_t stream) {
  cudaStreamSynchronize(stream);
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_status_host) return 0;
  int v = *(volatile int*)(g_status_host + dev);
  g_status_host[dev] = 0;
  return v;
}

}  // namespace tsb_host

namespace {

// split-K partial sums: library scratch keyed by (device, stream)
float* get_workspace(size_t bytes, cudaStream_t st) {
  return static_cast<float*>(tsb_scratch::get(st, tsb_scratch::GEMM_SPLITK, bytes, size_t(64) << 20));
}

int g_sm_count = 0;
int sm_count() {
  if (!g_sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

template <int BN, bool A_MN, bool B_MN>
int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_tf32_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return TSB_ERR_LAUNCH | ((int)cudaGetLastError() << 8);
    attr_set = true;
  }
  const long long items = (long long)p.tiles_m * p.tiles_n * p.batch * p.splits;
  const int grid = (int)(items < sm_count() ? items : sm_count());
  kern<<<grid, 192, C::SMEM_BYTES, st>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

template <int BN>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                   cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_tc<BN, false, false>(ta, tb, p, st);
  if (!a_mn && b_mn) return launch_tc<BN, false, true>(ta, tb, p, st);
  if (a_mn && !b_mn) return launch_tc<BN, true, false>(ta, tb, p, st);
  return launch_tc<BN, true, true>(ta, tb, p, st);
}

template <bool A_MN, bool B_MN>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  auto kern = gemm_tf32_pair_kernel<A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P2_SMEM_BYTES) != cudaSuccess)
      return TSB_ERR_LAUNCH | ((int)cudaGetLastError() << 8);
    attr_set = true;
  }
  const long long items = (long long)((p.m + 255) / 256) * ((p.n + P2_BN - 1) / P2_BN) * p.batch;
  long long pairs = sm_count() / 2;
  if (pairs > items) pairs = items;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = P2_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

// Copy of a [batch][rows][cols] operand whose row stride is not a multiple of four floats into a
// scratch array with the row stride rounded up (pad columns zero), so that TMA can address it.
__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int batch, int rows,
                                int cols, long long lds, long long ss, long long ldd, long long sd) {
  const long long total = (long long)batch * rows * ldd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int c, row;
    long long b;
    if ((total >> 32) == 0) {   // 32-bit divisions are several times cheaper
      const unsigned r = (unsigned)i / (unsigned)ldd;
      c = (int)((unsigned)i - r * (unsigned)ldd);
      const unsigned bb = r / (unsigned)rows;
      row = (int)(r - bb * (unsigned)rows);
      b = bb;
    } else {
      c = (int)(i % ldd);
      const long long r = i / ldd;
      row = (int)(r % rows);
      b = r / rows;
    }
    dst[b * sd + row * ldd + c] = c < cols ? src[b * ss + row * lds + c] : 0.f;
  }
}

float* pad_workspace(int slot, size_t bytes, cudaStream_t st) {
  return static_cast<float*>(tsb_scratch::get(st, slot ? tsb_scratch::GEMM_PAD_B : tsb_scratch::GEMM_PAD_A, bytes));
}

int dispatch_pair(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                  cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_pair<false, false>(ta, tb, p, st);
  if (!a_mn && b_mn) return launch_pair<false, true>(ta, tb, p, st);
  if (a_mn && !b_mn) return launch_pair<true, false>(ta, tb, p, st);
  return launch_pair<true, true>(ta, tb, p, st);
}

}  // namespace

// Chooses the split-K factor: enough work items to fill the SMs when the tile
// grid alone is small and K is long.
static int choose_splits(long long tiles, int kblocks, int forced) {
  if (forced > 0) return forced;
  const int sms = sm_count();
  if (tiles >= sms || kblocks < 16) return 1;
  long long s = sms / tiles;
  if (s > kblocks / 8) s = kblocks / 8;
  if (s > 32) s = 32;
  return s < 1 ? 1 : (int)s;
}

// Core entry shared by the allocating and the non-allocating front ends.
//   ws / ws_bytes : split-K scratch supplied by the caller (may be null when splits resolves to 1)
int tsb_gemm_tf32_impl(const float* a, const float* b, float* c, int m, int n, int k, long long lda,
                       long long ldb, long long ldc, int trans_a, int trans_b, int batch, long long sa,
                       long long sb, long long sc, int accumulate, int forced_splits, float* ws,
                       size_t ws_bytes, bool may_alloc, cudaStream_t st, int heads = 0, int head_mask = 0) {
  if (m <= 0 || n <= 0 || k <= 0 || batch <= 0) return TSB_ERR_ARG;
  if (heads < 0 || (heads > 0 && (batch % heads) != 0)) return TSB_ERR_ARG;
  if (heads == 0) head_mask = 0;
  const bool a_heads = (head_mask & 1) != 0, b_heads = (head_mask & 2) != 0, c_heads = (head_mask & 4) != 0;
  if (head_mask) forced_splits = 1;       // the split-K scratch and its reduction address C by one batch stride
  const bool aligned = (lda % 4 == 0) && (ldb % 4 == 0) && (sa % 4 == 0) && (sb % 4 == 0) &&
                       ((reinterpret_cast<uintptr_t>(a) & 15) == 0) && ((reinterpret_cast<uintptr_t>(b) & 15) == 0);
  // Only the row strides are off (e.g. 255-wide attention matrices): pad the operand rows into scratch
  // once (one pass over the operand) and run the tensor-core kernel on the padded copy.
  if (!aligned && may_alloc && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0) {
    const float* ap = a;
    const float* bp = b;
    long long lda2 = lda, ldb2 = ldb, sa2 = sa, sb2 = sb;
    const int rows_a = trans_a ? k : m, cols_a = trans_a ? m : k;
    const int rows_b = trans_b ? n : k, cols_b = trans_b ? k : n;
    bool okpad = true;
    if (((lda % 4) && a_heads) || ((ldb % 4) && b_heads)) return TSB_ERR_UNSUPPORTED;
    if ((lda % 4) || (batch > 1 && (sa % 4))) {
      lda2 = (cols_a + 3) / 4 * 4;
      sa2 = (long long)rows_a * lda2;
      float* buf = pad_workspace(0, (size_t)batch * sa2 * sizeof(float), st);
      if (!buf) okpad = false;
      else {
        const long long total = (long long)batch * rows_a * lda2;
        long long blocks = (total + 255) / 256;
        if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
        pad_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(a, buf, batch, rows_a, cols_a, lda, batch > 1 ? sa : 0, lda2,
                                                         sa2);
        ap = buf;
      }
    }
    if (okpad && ((ldb % 4) || (batch > 1 && (sb % 4)))) {
      ldb2 = (cols_b + 3) / 4 * 4;
      sb2 = (long long)rows_b * ldb2;
      float* buf = pad_workspace(1, (size_t)batch * sb2 * sizeof(float), st);
      if (!buf) okpad = false;
      else {
        const long long total = (long long)batch * rows_b * ldb2;
        long long blocks = (total + 255) / 256;
        if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
        pad_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(b, buf, batch, rows_b, cols_b, ldb, batch > 1 ? sb : 0, ldb2,
                                                         sb2);
        bp = buf;
      }
    }
    if (okpad)
      return tsb_gemm_tf32_impl(ap, bp, c, m, n, k, lda2, ldb2, ldc, trans_a, trans_b, batch, sa2, sb2, sc, accumulate,
                                forced_splits, ws, ws_bytes, may_alloc, st, heads,
                                head_mask & ~((ap != a ? 1 : 0) | (bp != b ? 2 : 0)));   // a padded copy is plain
  }
  if (!aligned && head_mask) return TSB_ERR_UNSUPPORTED;
  if (!aligned) {
    if (getenv("TSB_GEMM_TRACE"))
      fprintf(stderr, "[gemm] SIMT fallback m %d n %d k %d lda %lld ldb %lld ta %d tb %d batch %d sa %lld sb %lld a%%16 %d b%%16 %d\n",
              m, n, k, lda, ldb, trans_a, trans_b, batch, sa, sb, (int)(reinterpret_cast<uintptr_t>(a) & 15),
              (int)(reinterpret_cast<uintptr_t>(b) & 15));
    dim3 blk(16, 16), grd((n + 15) / 16, (m + 15) / 16, batch);
    gemm_simt_kernel<<<grd, blk, 0, st>>>(a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b, sa, sb, sc,
                                          accumulate);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
  }
  const int bn = n > 128 ? 256 : (n > 64 ? 128 : 64);
  GemmParams p;
  p.c = c; p.m = m; p.n = n; p.k = k; p.batch = batch; p.ldc = ldc; p.sc = sc;
  p.accumulate = accumulate;
  p.heads = head_mask ? heads : 0;
  p.a_heads = a_heads; p.b_heads = b_heads; p.c_heads = c_heads;
  p.a_shift = trans_a ? k : m;
  p.b_shift = trans_b ? n : k;
  p.sc2 = (long long)m * ldc;
  p.tiles_m = (m + BM - 1) / BM;
  p.tiles_n = (n + bn - 1) / bn;
  p.kblocks = (k + BK - 1) / BK;
  p.splits = choose_splits((long long)p.tiles_m * p.tiles_n * batch, p.kblocks, forced_splits);
  if (p.splits > p.kblocks) p.splits = p.kblocks;
  {   // no empty K ranges: re-derive the count from the per-split share
    const int per = (p.kblocks + p.splits - 1) / p.splits;
    p.splits = (p.kblocks + per - 1) / per;
  }
  p.ws = nullptr;
  p.status = tsb_host::status_word(st);
  if (!p.status) return TSB_ERR_LAUNCH;
  if (p.splits > 1) {
    const size_t need = (size_t)p.splits * batch * m * n * sizeof(float);
    if (ws && ws_bytes >= need) {
      p.ws = ws;
    } else if (may_alloc) {
      p.ws = get_workspace(need, st);
      if (!p.ws) return TSB_ERR_OOM;
    } else {
      return TSB_ERR_SCRATCH;
    }
  }
  // CTA pairs (256 x 256 tiles on SM pairs) when the problem has enough of them and no split-K
  bool use_pair = false;
  {
    const long long pair_items = (long long)((m + 255) / 256) * ((n + 255) / 256) * batch;
    const char* e = getenv("TSB_GEMM_PAIR");              // "0" selects the one-CTA tiles everywhere
    const bool enabled = !(e && e[0] == '0');
    use_pair = enabled && bn == 256 && p.splits == 1 && m >= 256 && pair_items * 4 >= sm_count() &&
               (!trans_a || m % 32 == 0) && (trans_b || n % 32 == 0);
  }
  const uint32_t bbox = use_pair ? P2_BNH : (uint32_t)bn;   // columns of B that one CTA stages
  // tensor maps (dims innermost first)
  CUtensorMap ta, tb;
  p.a_chunked = p.b_chunked = 0;
  const uint64_t sab = (uint64_t)(batch > 1 ? sa : (long long)(trans_a ? k : m) * lda) * 4;
  const uint64_t sbb = (uint64_t)(batch > 1 ? sb : (long long)(trans_b ? n : k) * ldb) * 4;
  int rc;
  // an operand in head layout: rows of all outer batches in the row dimension, the head as batch dimension
  const uint64_t outer = head_mask ? (uint64_t)(batch / heads) : 1;
  const uint64_t a_rows = a_heads ? outer : 1, a_bat = a_heads ? (uint64_t)heads : (uint64_t)batch;
  const uint64_t b_rows = b_heads ? outer : 1, b_bat = b_heads ? (uint64_t)heads : (uint64_t)batch;
  if (!trans_a) {   // A[m][k], K contiguous -> K-major
    uint64_t d[3] = {(uint64_t)k, (uint64_t)m * a_rows, a_bat}, s[2] = {(uint64_t)lda * 4, sab};
    uint32_t bx[3] = {BK, BM, 1};
    rc = tsb_host::make_tmap_f32(&ta, a, 3, d, s, bx);
  } else if (m % 32 == 0) {   // A stored [k][m], M contiguous -> MN-major; all chunks of a stage in one box
    uint64_t d[4] = {32, (uint64_t)k * a_rows, (uint64_t)m / 32, a_bat}, s[3] = {(uint64_t)lda * 4, 128, sab};
    uint32_t bx[4] = {32, BK, BM / 32, 1};
    rc = tsb_host::make_tmap_f32(&ta, a, 4, d, s, bx, true);
    p.a_chunked = 1;
  } else {
    uint64_t d[3] = {(uint64_t)m, (uint64_t)k * a_rows, a_bat}, s[2] = {(uint64_t)lda * 4, sab};
    uint32_t bx[3] = {32, BK, 1};
    rc = tsb_host::make_tmap_f32(&ta, a, 3, d, s, bx, true);
  }
  if (rc) return rc;
  if (trans_b) {    // B stored [n][k], K contiguous -> K-major
    uint64_t d[3] = {(uint64_t)k, (uint64_t)n * b_rows, b_bat}, s[2] = {(uint64_t)ldb * 4, sbb};
    uint32_t bx[3] = {BK, bbox, 1};
    rc = tsb_host::make_tmap_f32(&tb, b, 3, d, s, bx);
  } else if (n % 32 == 0) {   // B[k][n], N contiguous -> MN-major; all chunks of a stage in one box
    uint64_t d[4] = {32, (uint64_t)k * b_rows, (uint64_t)n / 32, b_bat}, s[3] = {(uint64_t)ldb * 4, 128, sbb};
    uint32_t bx[4] = {32, BK, bbox / 32, 1};
    rc = tsb_host::make_tmap_f32(&tb, b, 4, d, s, bx, true);
    p.b_chunked = 1;
  } else {
    uint64_t d[3] = {(uint64_t)n, (uint64_t)k * b_rows, b_bat}, s[2] = {(uint64_t)ldb * 4, sbb};
    uint32_t bx[3] = {32, BK, 1};
    rc = tsb_host::make_tmap_f32(&tb, b, 3, d, s, bx, true);
  }
  if (rc) return rc;
  const bool a_mn = trans_a != 0, b_mn = trans_b == 0;
  if (use_pair) rc = dispatch_pair(a_mn, b_mn, ta, tb, p, st);
  else if (bn == 256) rc = dispatch_major<256>(a_mn, b_mn, ta, tb, p, st);
  else if (bn == 128) rc = dispatch_major<128>(a_mn, b_mn, ta, tb, p, st);
  else rc = dispatch_major<64>(a_mn, b_mn, ta, tb, p, st);
  if (rc) return rc;
  if (p.splits > 1) {
    const long long per_split = (long long)batch * m * n;
    int blocks = (int)((per_split + 255) / 256);
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, st>>>(p.ws, c, p.splits, per_split, m, n, ldc, sc, accumulate);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
  }
  const int late = tsb_host::peek_status();
  return late ? TSB_ERR_TIMEOUT | (late << 8) : TSB_OK;
}

extern "C" {

int tsb_gemm_tf32(const float* a, const float* b, float* c, int m, int n, int k, long long lda, long long ldb,
                  long long ldc, int trans_a, int trans_b, int batch, long long sa, long long sb, long long sc,
                  int accumulate, void* stream) {
  return tsb_gemm_tf32_impl(a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b, batch, sa, sb, sc, accumulate, 0,
                            nullptr, 0, true, static_cast<cudaStream_t>(stream));
}

// Batched GEMM over (outer, head) with operands in head layout.  batch = outer * heads; bit 0 / 1 / 2 of
// head_mask says that A / B / C is stored [outer][row][head][col] (what a [N, T, heads * d] projection output is,
// read in place) instead of [outer][head][row][col]: such an operand is given with its row stride (heads * d), its
// HEAD stride as batch stride (d), and rows-per-outer-batch equal to its full row extent.  An operand in head layout
// whose row dimension is K (an MN-major operand) is read past the end of its K rows into the next outer batch when
// K is not a multiple of 32; the other operand is zero there, so finite data there contributes nothing.
int tsb_gemm_tf32_heads(const float* a, const float* b, float* c, int m, int n, int k, long long lda, long long ldb,
                        long long ldc, int trans_a, int trans_b, int batch, long long sa, long long sb, long long sc,
                        int accumulate, int heads, int head_mask, void* stream) {
  if (heads <= 0 || (head_mask & ~7)) return TSB_ERR_ARG;
  if ((head_mask & 1) && (head_mask & 2) && trans_a && !trans_b) return TSB_ERR_UNSUPPORTED;   // both K dimensions folded
  return tsb_gemm_tf32_impl(a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b, batch, sa, sb, sc, accumulate, 1,
                            nullptr, 0, true, static_cast<cudaStream_t>(stream), heads, head_mask);
}

// Same with an explicit split-K factor (tests, tuning).
int tsb_gemm_tf32_splitk(const float* a, const float* b, float* c, int m, int n, int k, long long lda,
                         long long ldb, long long ldc, int trans_a, int trans_b, int splits, void* stream) {
  return tsb_gemm_tf32_impl(a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b, 1, 0, 0, 0, 0, splits, nullptr, 0,
                            true, static_cast<cudaStream_t>(stream));
}

// Synchronise the stream and return (then clear) the device-side wait status:
// 0 = clean, otherwise the code of the wait that ran out.
int tsb_device_status(void* stream) { return tsb_host::read_status(static_cast<cudaStream_t>(stream)); }

}  // extern "C"
