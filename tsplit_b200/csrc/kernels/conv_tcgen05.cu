// Implicit-GEMM 2-D convolution on the 5th-generation tensor cores (sm_100a),
// TF32 inputs / fp32 accumulate in TMEM, channels-last operands:
//   mode 0  forward : y[n,oh,ow,o]  = sum_{kh,kw,c} x[n,oh*s-ph+kh,ow*s-pw+kw,c] * w[o,kh,kw,c]
//   mode 1  dgrad   : dx[n,ih,iw,c] = sum_{kh,kw,o} dy[n,(ih+ph-kh)/s,(iw+pw-kw)/s,o] * w[o,kh,kw,c]
//   mode 2  wgrad   : dw[o,kh,kw,c] = sum_{n,oh,ow} dy[n,oh,ow,o] * x[n,oh*s-ph+kh,ow*s-pw+kw,c]
//
// No im2col buffer exists anywhere.  The patch operand is gathered straight into
// swizzled shared memory by eight cp.async producer warps (zero-fill for padding
// and tails); the dense operand (filters, or dy for wgrad) arrives by TMA; one
// elected thread issues tcgen05.mma.kind::tf32 into double-buffered TMEM
// accumulators; four epilogue warps drain TMEM to global while the next tile is
// being multiplied.  wgrad splits its long reduction (all output pixels) across
// CTAs and reduces the partial sums in a fixed order.
//
// Role in the reference: cudnnConvolutionForward / BackwardData / BackwardFilter
// (src/ops/CudnnConv2d.cu:127-602).
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"
#include "scratch.h"

using namespace tsb;

namespace {

constexpr int BM = 128;
constexpr int BK = 32;
constexpr int UMMA_K = 8;
constexpr int A_STAGE_BYTES = BM * BK * 4;
constexpr int STORE_STAGING_BYTES = 4 * 2048;   // per epilogue warp: 32 rows x 16 columns on their way to a TMA store
constexpr int GATHER_WARPS = 8;        // two per scheduler, so one warp's address arithmetic hides the other's
constexpr int GATHER_THREADS = GATHER_WARPS * 32;
constexpr int NUM_THREADS = 6 * 32 + GATHER_THREADS;   // warp0 TMA, warp1 MMA, warps2-5 epilogue, then gather

struct ConvParams {
  const float* src;    // gathered tensor: x (fwd, wgrad) or dy (dgrad)
  float* out;
  float* ws;
  int N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride;
  int M;               // GEMM rows
  int NC;              // GEMM columns of one column group
  int K;               // fwd: KH*KW*C
  int kblocks;         // k-blocks of one full reduction
  int ocb;             // dgrad: ceil(O/32) k-blocks per filter tap
  int tiles_m, tiles_n, taps;   // taps = KH*KW column groups (wgrad), else 1
  int splits;
  int accumulate;
  long long ldc;
  int tma_store;       // the output tile leaves through shared memory and TMA stores (map `tmo`)
  float* stats;        // forward only, may be null: per-CTA column sums / sums of squares of the output
  long long stats_plane;   // floats between the plane of sums and the plane of sums of squares
  int a3d;             // wgrad: dy arrives through the 3-D (32 channels, pixel, chunk) view
  int* status;
  unsigned long long* prof;   // role-time counters (only written when built with -DTSB_CONV_PROF)
};

// Narrow tiles (BN <= 128) of the TMA-only kernels run two CTAs per SM: a stage's four MMAs cost
// the single issuing thread about as much time for a 64-wide tile as for a 256-wide one, so a second
// CTA's issue thread fills the tensor pipe that one CTA leaves idle.  Each of the two gets half the
// stages (2 x ~97 KB of shared memory) and its own TMEM columns (2 x 128 or 2 x 256 of 512).
template <int BN, bool IM2COL>
struct Cfg {
  static constexpr int OCC = (IM2COL && BN <= 128) ? 2 : 1;       // CTAs per SM
  static constexpr int B_STAGE_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = ((BN == 256) ? 4 : (BN == 128 ? 6 : 8)) / OCC;
  static constexpr int STAT_BYTES = 4 * 2 * BN * 4;          // per epilogue warp: (sum, sum of squares) per tile column
  static constexpr int SMEM_BYTES = STORE_STAGING_BYTES + STAT_BYTES + STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
// Arrival on `bar` that the hardware performs once every cp.async issued so far by this thread has
// written shared memory.  `.noinc`: the barrier's expected count already includes this arrival.
// The tensor core may read the stage as soon as the barrier's phase completes; no proxy fence
// stands between the copies and the MMA (same protocol as CUTLASS's sm100 cp.async mainloop,
// cutlass/gemm/collective/sm100_mma_cpasync_warpspecialized.hpp).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Developer diagnostic: with -DTSB_CONV_PROF each role adds the cycles it spent waiting / working to
// sixteen global counters, and the host prints them per CTA after every launch (which it then
// synchronises).  Off by default: the macros expand to nothing.
#ifdef TSB_CONV_PROF
#define PROF_DECL(n) long long prof_##n = 0
#define PROF_BEGIN(n) const long long prof_t_##n = clock64()
#define PROF_END(n) prof_##n += clock64() - prof_t_##n
#define PROF_FLUSH(idx, n) atomicAdd(&p.prof[idx], (unsigned long long)prof_##n)
#else
#define PROF_DECL(n)
#define PROF_BEGIN(n)
#define PROF_END(n)
#define PROF_FLUSH(idx, n)
#endif

// ---- column statistics of the output, taken in the epilogue (for a batch norm that follows) -------
// The 32 x 16 block that a warp has parked in its staging buffer (64-byte rows, 64B swizzle) is read
// back column-wise: lanes 0-15 take rows 0-15 of column (lane & 15), lanes 16-31 rows 16-31, the two
// halves meet by shuffle and lanes 0-15 add (sum, sum of squares) to the warp's accumulators in
// shared memory.  Rows past the end of the tensor hold zeros (their patches were zero-filled) and
// add nothing.  Tiles are visited in a fixed order, so the result does not depend on scheduling.
__device__ __forceinline__ void stat_accumulate(const uint8_t* stg, float* acc, int colbase, int lane) {
  const int colh = lane & 15, rh = lane >> 4;
  const uint32_t base = smem_u32(stg) + (uint32_t)(colh & 3) * 4;
  const uint32_t c4 = (uint32_t)(colh >> 2);
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const uint32_t row = (uint32_t)(rh * 16 + r);
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(base + row * 64 + ((c4 ^ ((row >> 1) & 3)) << 4)) : "memory");
    s += v;
    ss += v * v;
  }
  s += __shfl_xor_sync(0xffffffffu, s, 16);
  ss += __shfl_xor_sync(0xffffffffu, ss, 16);
  if (lane < 16) {
    acc[2 * (colbase + lane)] += s;
    acc[2 * (colbase + lane) + 1] += ss;
  }
}
// After the last tile: the four epilogue warps (128 threads, named barrier 1) add their accumulators
// in warp order and write the CTA's partial sums for its column tile to slot `slot` of the two planes.
__device__ __forceinline__ void stat_flush(const ConvParams& p, const float* stat, int bn, int q, int lane, int slot,
                                           int col0) {
  asm volatile("bar.sync 1, 128;" ::: "memory");
  for (int col = q * 32 + lane; col < bn; col += 128) {
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      s += stat[w * 2 * bn + 2 * col];
      ss += stat[w * 2 * bn + 2 * col + 1];
    }
    const int gc = col0 + col;
    if (gc < p.NC) {
      p.stats[(long long)slot * p.NC + gc] = s;
      p.stats[p.stats_plane + (long long)slot * p.NC + gc] = ss;
    }
  }
}

struct Item {
  int m0, n0, tap, split, kb0, kb1;
};

__device__ __forceinline__ Item decode_item(const ConvParams& p, long long item, int BN_) {
  Item it;
  const int tiles = p.tiles_m * p.tiles_n * p.taps;
  const int tile = (int)(item % tiles);
  it.split = (int)(item / tiles);
  const int per_m = p.tiles_n * p.taps;
  it.m0 = (tile / per_m) * BM;
  const int r = tile % per_m;
  it.tap = r / p.tiles_n;
  it.n0 = (r % p.tiles_n) * BN_;
  const int per = (p.kblocks + p.splits - 1) / p.splits;
  it.kb0 = it.split * per;
  it.kb1 = min(p.kblocks, it.kb0 + per);
  return it;
}

// IM2COL: the patch operand also arrives by TMA (im2col-mode tensor map `tmi`), so the CTA has no
// gather warps at all; needs the gathered tensor's channel count to be a multiple of 32 and is not
// used for strided dgrad.  Otherwise the eight cp.async warps below gather it.
template <int MODE, int BN, bool IM2COL>
__global__ void __launch_bounds__(IM2COL ? (MODE == 2 ? 288 : 192) : NUM_THREADS, Cfg<BN, IM2COL>::OCC)
conv_tf32_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmi,
                 const __grid_constant__ CUtensorMap tmo, const ConvParams p) {
  using C = Cfg<BN, IM2COL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_stg = smem;
  float* smem_stat = reinterpret_cast<float*>(smem + STORE_STAGING_BYTES);
  uint8_t* smem_a = smem + STORE_STAGING_BYTES + C::STAT_BYTES;
  uint8_t* smem_b = smem_a + C::STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_a + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], IM2COL ? 1 : 1 + GATHER_THREADS);   // TMA expect_tx arrive (+ one arrive per gather thread)
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm);
    if (IM2COL) tma_prefetch_desc(&tmi);
    if (p.tma_store) tma_prefetch_desc(&tmo);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const long long items = (long long)p.tiles_m * p.tiles_n * p.taps * p.splits;
  // which shared-memory operand the TMA fills / the gather warps fill
  constexpr bool TMA_IS_A = (MODE == 2);
  constexpr int TMA_BYTES = TMA_IS_A ? A_STAGE_BYTES : C::B_STAGE_BYTES;

  // wgrad with both operands by TMA.  Issuing a TMA costs the issuing thread on the order of a
  // hundred cycles, and a k-block needs up to nine boxes, so four producer threads (one lane each
  // of warp 0 and of the three extra warps) share them: producer q fetches chunks q and q+4 of the
  // patch tile (a chunk = 32 pixels x 32 channels of the filter tap its columns belong to), and
  // producer 0 also posts the byte count and fetches the dy tile.  Transfers of the other
  // producers may complete before producer 0 posts the count; the barrier's phase cannot complete
  // before that arrival.
  auto wgrad_producer = [&](int q) {
    constexpr int NCH = BN / 32;
    uint32_t it = 0;
    bool ok = true;
    PROF_DECL(tw); PROF_DECL(tt);
    PROF_BEGIN(tt);
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const Item w = decode_item(p, item, BN);
      int c0[2], kh[2], kw[2];
      bool cv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int ci = q + 4 * u;
        const int col = w.n0 + ci * 32;
        cv[u] = ci < NCH && col < p.NC;
        const int tap = col / p.C;
        c0[u] = col - tap * p.C;
        kh[u] = tap / p.KW; kw[u] = tap - kh[u] * p.KW;
      }
      int nv = (p.NC - w.n0 + 31) / 32;
      if (nv > NCH) nv = NCH;
      const uint32_t tx = A_STAGE_BYTES + nv * (BK * 128);
      // position of the first pixel of the first k-block
      const int pix0 = w.kb0 * BK;
      int n = pix0 / (p.OH * p.OW);
      const int rem = pix0 - n * (p.OH * p.OW);
      int oy = rem / p.OW, ox = rem - oy * p.OW;
      for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        PROF_BEGIN(tw);
        if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x207 + q)) { ok = false; break; }
        PROF_END(tw);
        if (q == 0) {
          mbar_expect_tx(&full[s], tx);
          if (p.a3d) {           // dy viewed (32 channels, pixel, channel chunk): four chunks in one box
            tma_load_3d(smem_a + s * A_STAGE_BYTES, &tm, &full[s], 0, kb * BK, w.m0 >> 5);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              tma_load_2d(smem_a + s * A_STAGE_BYTES + c * (BK * 128), &tm, &full[s], w.m0 + c * 32, kb * BK);
          }
        }
        const int bw = ox * p.stride - p.pw, bh = oy * p.stride - p.ph;
#pragma unroll
        for (int u = 0; u < 2; ++u)
          if (cv[u])
            tma_load_im2col_4d(smem_b + s * C::B_STAGE_BYTES + (q + 4 * u) * (BK * 128), &tmi, &full[s], c0[u], bw,
                               bh, n, (uint16_t)kw[u], (uint16_t)kh[u]);
        ox += BK;
        while (ox >= p.OW) { ox -= p.OW; ++oy; }
        while (oy >= p.OH) { oy -= p.OH; ++n; }
      }
    }
    PROF_END(tt);
    if (q == 0) { PROF_FLUSH(4, tw); PROF_FLUSH(5, tt); }
    if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (IM2COL && MODE == 0) {
      // forward with both operands by TMA: one im2col box (128 pixels x 32 channels of one filter
      // tap) and one weight box per k-block; k runs over (tap, 32-channel block)
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        PROF_DECL(tw); PROF_DECL(tt);
        PROF_BEGIN(tt);
        const int cpb = p.C >> 5;
        for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
          const Item w = decode_item(p, item, BN);
          const int n = w.m0 / (p.OH * p.OW);
          const int rem = w.m0 - n * (p.OH * p.OW);
          const int oy = rem / p.OW, ox = rem - oy * p.OW;
          const int bw = ox * p.stride - p.pw, bh = oy * p.stride - p.ph;   // base position of the first pixel
          int tap = w.kb0 / cpb, cb = w.kb0 - tap * cpb;
          int kh = tap / p.KW, kw = tap - kh * p.KW;
          for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1;
            PROF_BEGIN(tw);
            if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x201)) { ok = false; break; }
            PROF_END(tw);
            mbar_expect_tx(&full[s], C::STAGE_BYTES);
            tma_load_im2col_4d(smem_a + s * A_STAGE_BYTES, &tmi, &full[s], cb * 32, bw, bh, n, (uint16_t)kw,
                               (uint16_t)kh);
            tma_load_2d(smem_b + s * C::B_STAGE_BYTES, &tm, &full[s], kb * BK, w.n0);
            if (++cb == cpb) {
              cb = 0;
              if (++kw == p.KW) { kw = 0; ++kh; }
            }
          }
        }
        PROF_END(tt);
        PROF_FLUSH(4, tw); PROF_FLUSH(5, tt);
        if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    } else if (IM2COL && MODE == 2) {
      if (lane == 0) wgrad_producer(0);
    } else if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      PROF_DECL(tw); PROF_DECL(tt);
      PROF_BEGIN(tt);
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const Item w = decode_item(p, item, BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          PROF_BEGIN(tw);
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x201)) { ok = false; break; }
          PROF_END(tw);
          mbar_expect_tx(&full[s], TMA_BYTES);
          if (MODE == 0) {          // filters [O][K], K-major
            tma_load_2d(smem_b + s * C::B_STAGE_BYTES, &tm, &full[s], kb * BK, w.n0);
          } else if (MODE == 1) {   // filters viewed (C, tap, O): MN-major chunks of 32 channels
            const int tap = kb / p.ocb, o0 = (kb % p.ocb) * BK;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              tma_load_3d(smem_b + s * C::B_STAGE_BYTES + c * (BK * 128), &tm, &full[s], w.n0 + c * 32, tap, o0);
          } else {                  // dy [pixels][O]: MN-major chunks of 32 output channels
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              tma_load_2d(smem_a + s * A_STAGE_BYTES + c * (BK * 128), &tm, &full[s], w.m0 + c * 32, kb * BK);
          }
        }
      }
      PROF_END(tt);
      PROF_FLUSH(4, tw); PROF_FLUSH(5, tt);
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr int A_MN = (MODE == 2) ? 1 : 0;
      constexpr int B_MN = (MODE == 0) ? 0 : 1;
      constexpr uint32_t idesc = make_idesc_tf32(BM, BN, A_MN, B_MN);
      // shared-memory descriptors: MN-major operands use the 32-byte-atom 128B swizzle (chunks of 32
      // columns BK*128 bytes apart, 1024 bytes per K step), K-major ones the plain 128B swizzle
      constexpr uint32_t A_HI = A_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t B_HI = B_MN ? smem_desc_hi(512, LAYOUT_SW128_BASE32B) : smem_desc_hi(1024);
      constexpr uint32_t A_KSTEP = (A_MN ? 1024 : UMMA_K * 4) >> 4, B_KSTEP = (B_MN ? 1024 : UMMA_K * 4) >> 4;
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), A_MN ? BK * 128 : 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), B_MN ? BK * 128 : 16);
      uint32_t it = 0, acc_it = 0;
      bool ok = true, ready = false;
      PROF_DECL(mf); PROF_DECL(me); PROF_DECL(mi); PROF_DECL(mt); PROF_DECL(mm); PROF_DECL(mc);
      PROF_BEGIN(mt);
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++acc_it) {
        const Item w = decode_item(p, item, BN);
        const int acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        PROF_BEGIN(me);
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, 0x202)) { ok = false; break; }
        PROF_END(me);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          PROF_BEGIN(mf);
          if (!ready && !mbar_wait(&full[s], ph, p.status, 0x203)) { ok = false; break; }
          PROF_END(mf);
          PROF_BEGIN(mi);
          {   // probe the next stage now; the answer arrives while this stage's MMAs are issued
            const uint32_t it2 = it + 1;
            ready = mbar_test(&full[it2 % C::STAGES], (it2 / C::STAGES) & 1);
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (C::B_STAGE_BYTES >> 4);
          PROF_BEGIN(mm);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_tf32(d_tmem, smem_desc_join(A_HI, a_lo + k * A_KSTEP), smem_desc_join(B_HI, b_lo + k * B_KSTEP),
                      idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          PROF_END(mm);
          PROF_BEGIN(mc);
          umma_commit(&empty[s]);
          PROF_END(mc);
          PROF_END(mi);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
      PROF_END(mt);
      PROF_FLUSH(0, mf); PROF_FLUSH(1, me); PROF_FLUSH(2, mi); PROF_FLUSH(3, mt); PROF_FLUSH(13, mm); PROF_FLUSH(14, mc);
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    float* my_stat = smem_stat + q * 2 * BN;
    if (MODE == 0 && p.stats)
      for (int i = lane; i < 2 * BN; i += 32) my_stat[i] = 0.f;
    PROF_DECL(ew); PROF_DECL(et);
    PROF_BEGIN(et);
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++acc_it) {
      const Item w = decode_item(p, item, BN);
      const int acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      const bool has_k = w.kb0 < w.kb1;
      PROF_BEGIN(ew);
      if (!mbar_wait(&tfull[acc], acc_ph, p.status, 0x204)) { ok = false; break; }
      PROF_END(ew);
      tc_fence_after();
      const int row = w.m0 + q * 32 + lane;
      const long long coloff = (MODE == 2) ? (long long)w.tap * p.C : 0;
      float* crow;
      bool accumulate;
      if (p.splits > 1) {
        crow = p.ws + ((long long)w.split * p.M + row) * p.ldc + coloff;
        accumulate = false;
      } else {
        crow = p.out + (long long)row * p.ldc + coloff;
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
        const int col = w.n0 + c0;
        if (p.tma_store) {
          // Each lane holds one output row; written straight to global that is 32 scattered 16-byte
          // pieces per instruction.  Instead the warp parks 32 rows x 16 columns in shared memory
          // (64-byte rows, 64B swizzle: conflict-free) and one TMA store writes them as full lines;
          // the TMA unit also clips rows / columns that lie outside the tensor.
          uint8_t* stg = smem_stg + q * 2048;
          const uint32_t srow = smem_u32(stg) + lane * 64;
          const uint32_t sx = (uint32_t)(lane >> 1) & 3;
          const int row0 = w.m0 + q * 32;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (lane == 0) bulk_wait_read();       // the previous store has finished reading the buffer
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int j = half * 16 + c * 4;
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(srow + (((uint32_t)c ^ sx) << 4)),
                           "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                           : "memory");
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row0 < p.M && col + half * 16 < p.NC) {
              tma_store_2d(&tmo, stg, col + half * 16, row0);
              bulk_commit();
            }
            if (MODE == 0 && p.stats) stat_accumulate(stg, my_stat, c0 + half * 16, lane);
          }
          continue;
        }
        if (row < p.M && col < p.NC) {
          float* dst = crow + col;
          const bool vec_ok = (col + 32 <= p.NC) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
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
              if (col + j < p.NC) dst[j] = accumulate ? dst[j] + v[j] : v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (p.tma_store && lane == 0) bulk_wait_all();     // this lane's stores are complete before the CTA exits
    if (MODE == 0 && p.stats)            // grid is a multiple of tiles_n: this CTA saw one column tile only
      stat_flush(p, smem_stat, BN, q, lane, blockIdx.x / p.tiles_n, (blockIdx.x % p.tiles_n) * BN);
    PROF_END(et);
    if (warp == 2 && lane == 0) { PROF_FLUSH(11, ew); PROF_FLUSH(12, et); }
  } else if (IM2COL) {
    // ---------------------------------------------------------------- extra TMA producers (wgrad only)
    if (MODE == 2 && lane == 0) wgrad_producer(warp - 5);
  } else {
    // ---------------------------------------------------------------- gather producers (warps 6..)
    // The loop over k-blocks is kept short on purpose: with few warps per scheduler the chain of
    // dependent address instructions, not the memory system, bounds the rate of k-blocks.  So
    // everything that depends only on the tile (row origins, which filter taps fall inside the
    // image, shared-memory offsets) is computed once per tile, and the (tap, channel) position
    // advances incrementally instead of being divided out of k.
    const int t = threadIdx.x - 6 * 32;       // 0..GATHER_THREADS-1
    uint32_t it = 0;                          // k-blocks issued by this thread
    bool ok = true;
    PROF_DECL(ge); PROF_DECL(gt);
    PROF_BEGIN(gt);
    const int ntaps = p.KH * p.KW;
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const Item w = decode_item(p, item, BN);
      if (MODE == 0 || MODE == 1) {
        // A tile: 128 rows (pixels) x 32 k, K-major, 128B swizzle.  Thread owns 16B chunk j of rows rg+32i.
        constexpr int RPT = BM / (GATHER_THREADS / 8);   // rows per thread
        constexpr int RSTEP = GATHER_THREADS / 8;
        const int j = t & 7, rg = t >> 3;
        const uint32_t soff = (uint32_t)(rg * 128 + ((j ^ (rg & 7)) << 4));   // (rg + RSTEP*i) & 7 == rg & 7
        const int PH = (MODE == 0) ? p.OH : p.H, PW = (MODE == 0) ? p.OW : p.W;   // pixel grid of the rows
        const int SH = (MODE == 0) ? p.H : p.OH, SW = (MODE == 0) ? p.W : p.OW;   // grid of the gathered tensor
        const int SC = (MODE == 0) ? p.C : p.O;                                   // its channel count
        const bool masked = ntaps <= 64 && (MODE == 0 || p.stride == 1);
        const float* rowptr[RPT];      // origin of the row's patch (may point outside; never read when invalid)
        int a0[RPT], b0[RPT];
        unsigned long long vmask[RPT]; // bit tap = that filter tap reads inside the image for this row
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int pix = w.m0 + rg + RSTEP * i;
          vmask[i] = 0;
          if (pix < p.M) {
            const int n = pix / (PH * PW);
            const int rem = pix - n * (PH * PW);
            const int y = rem / PW, x = rem - y * PW;
            if (MODE == 0) { a0[i] = y * p.stride - p.ph; b0[i] = x * p.stride - p.pw; }
            else           { a0[i] = y + p.ph;            b0[i] = x + p.pw; }
            if (MODE == 0 || p.stride == 1)
              rowptr[i] = p.src + (((long long)n * SH + a0[i]) * SW + b0[i]) * SC;
            else
              rowptr[i] = p.src + (long long)n * SH * SW * SC;
            if (masked) {
              unsigned long long colm = 0;
              for (int kw = 0; kw < p.KW; ++kw) {
                const int xx = (MODE == 0) ? b0[i] + kw : b0[i] - kw;
                if ((unsigned)xx < (unsigned)SW) colm |= 1ull << kw;
              }
              for (int kh = 0; kh < p.KH; ++kh) {
                const int yy = (MODE == 0) ? a0[i] + kh : a0[i] - kh;
                if ((unsigned)yy < (unsigned)SH) vmask[i] |= colm << (kh * p.KW);
              }
            }
          } else {
            rowptr[i] = p.src; a0[i] = -(1 << 28); b0[i] = -(1 << 28);
          }
        }
        // (tap, channel) position of this thread's chunk at the first k-block
        int tap, kh, kw, ch, ob = 0;
        if (MODE == 0) {
          const int k = w.kb0 * BK + j * 4;
          tap = k / p.C; ch = k - tap * p.C;
        } else {
          tap = w.kb0 / p.ocb; ob = w.kb0 - tap * p.ocb;
          ch = ob * BK + j * 4;
        }
        kh = tap / p.KW; kw = tap - kh * p.KW;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          PROF_BEGIN(ge);
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x205)) { ok = false; break; }
          PROF_END(ge);
          const bool kvalid = (MODE == 0) ? (tap < ntaps) : (ch < p.O);
          // element offset of this k-chunk relative to the row origin
          const int delta = (MODE == 0) ? (kh * SW + kw) * SC + ch : -((kh * SW + kw) * SC) + ch;
          const uint32_t sdst = smem_u32(smem_a + s * A_STAGE_BYTES) + soff;
          if (masked) {
            const int sh = tap & 63;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
              const bool v = kvalid && ((vmask[i] >> sh) & 1ull);
              cp_async16(sdst + i * (RSTEP * 128), v ? rowptr[i] + delta : p.src, v);
            }
          } else {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
              bool v = kvalid;
              const float* src;
              if (MODE == 0) {
                v = v && (unsigned)(a0[i] + kh) < (unsigned)SH && (unsigned)(b0[i] + kw) < (unsigned)SW;
                src = rowptr[i] + delta;
              } else if (p.stride == 1) {
                v = v && (unsigned)(a0[i] - kh) < (unsigned)SH && (unsigned)(b0[i] - kw) < (unsigned)SW;
                src = rowptr[i] + delta;
              } else {
                const int ty = a0[i] - kh, tx = b0[i] - kw;
                const int yy = ty / p.stride, xx = tx / p.stride;
                v = v && ty >= 0 && tx >= 0 && (yy * p.stride == ty) && (xx * p.stride == tx) &&
                    yy < SH && xx < SW;
                src = rowptr[i] + ((long long)yy * SW + xx) * SC + ch;
              }
              cp_async16(sdst + i * (RSTEP * 128), v ? src : p.src, v);
            }
          }
          cp_async_arrive(&full[s]);     // this thread's arrival fires when its copies above have landed
          // advance to the next k-block
          if (MODE == 0) {
            ch += BK;
            while (ch >= p.C) {
              ch -= p.C; ++tap;
              if (++kw == p.KW) { kw = 0; ++kh; }
            }
          } else {
            ch += BK;
            if (++ob == p.ocb) {
              ob = 0; ch = j * 4; ++tap;
              if (++kw == p.KW) { kw = 0; ++kh; }
            }
          }
        }
      } else {
        // wgrad B tile: 32 rows (pixels = k) x BN columns, MN-major, 128B swizzle with 32B atoms.
        // Columns are the flattened (tap, channel) index, so one tile spans several filter taps and
        // the dy tile is shared between them.  Thread owns pixel row t/8 and 16-byte piece t%8 of
        // every 32-column chunk, so its swizzled position inside a chunk is a per-thread constant.
        constexpr int PPT = BN / 32;           // pieces per thread = 32-column chunks of the tile
        const int kr = t >> 3, sub = t & 7;
        const int mpix = p.N * p.OH * p.OW;
        const bool masked = ntaps <= 64;
        int poff[PPT];                         // element offset of the piece relative to the row's origin
        int ptap[PPT];                         // filter tap of the piece, or -1 when the column is out of range
#pragma unroll
        for (int i = 0; i < PPT; ++i) {
          const int col = w.n0 + i * 32 + sub * 4;
          if (col < p.NC) {
            const int tap = col / p.C, ch = col - tap * p.C;
            const int kh = tap / p.KW, kw = tap - kh * p.KW;
            ptap[i] = tap;
            poff[i] = (kh * p.W + kw) * p.C + ch;
          } else {
            ptap[i] = -1; poff[i] = 0;
          }
        }
        // pixel state of this thread's row at the first k-block
        int pix = w.kb0 * BK + kr;
        int n = pix / (p.OH * p.OW);
        int rem = pix - n * (p.OH * p.OW);
        int oy = rem / p.OW, ox = rem - oy * p.OW;
        const uint32_t piece = ((((uint32_t)sub >> 1) ^ (uint32_t)(kr & 3)) << 1) | ((uint32_t)sub & 1);
        const uint32_t soff = (uint32_t)(kr * 128) + (piece << 4);
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          PROF_BEGIN(ge);
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x206)) { ok = false; break; }
          PROF_END(ge);
          const uint32_t sdst = smem_u32(smem_b + s * C::B_STAGE_BYTES) + soff;
          const int y0 = oy * p.stride - p.ph, x0 = ox * p.stride - p.pw;
          const bool pvalid = pix < mpix;
          const float* rowptr = p.src + (((long long)n * p.H + y0) * p.W + x0) * p.C;
          if (masked) {
            unsigned long long tapmask = 0;    // bit tap = that tap of this pixel reads inside the image
            if (pvalid) {
              unsigned long long colm = 0;
              for (int kw = 0; kw < p.KW; ++kw)
                if ((unsigned)(x0 + kw) < (unsigned)p.W) colm |= 1ull << kw;
              for (int kh = 0; kh < p.KH; ++kh)
                if ((unsigned)(y0 + kh) < (unsigned)p.H) tapmask |= colm << (kh * p.KW);
            }
#pragma unroll
            for (int i = 0; i < PPT; ++i) {
              const bool v = ptap[i] >= 0 && ((tapmask >> (ptap[i] & 63)) & 1ull);
              cp_async16(sdst + i * (BK * 128), v ? rowptr + poff[i] : p.src, v);
            }
          } else {
#pragma unroll
            for (int i = 0; i < PPT; ++i) {
              const int kh = ptap[i] / p.KW, kw = ptap[i] - kh * p.KW;
              const bool v = pvalid && ptap[i] >= 0 && (unsigned)(y0 + kh) < (unsigned)p.H &&
                             (unsigned)(x0 + kw) < (unsigned)p.W;
              cp_async16(sdst + i * (BK * 128), v ? rowptr + poff[i] : p.src, v);
            }
          }
          cp_async_arrive(&full[s]);     // this thread's arrival fires when its copies above have landed
          // advance the pixel by one k-block
          pix += BK; ox += BK;
          while (ox >= p.OW) { ox -= p.OW; ++oy; }
          while (oy >= p.OH) { oy -= p.OH; ++n; }
        }
      }
    }
    cp_async_wait_all();                     // nothing of this thread is in flight when the CTA exits
    PROF_END(gt);
    if (warp == 6 && lane == 0) { PROF_FLUSH(6, ge); PROF_FLUSH(9, gt); }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair forward kernel (cta_group::2): a cluster of two CTAs on an SM pair computes 256 pixels x
// 256 output channels.  Each CTA stages the im2col box of its own 128 pixels and its own 128 filter
// rows (32 KB per k-block instead of 48 KB: six stages, and the filters cross L2 -> SM once per
// pair); the leader's elected thread issues 256 x 256 x 8 MMAs that run on both SMs; each CTA
// drains and stores its own 128 x 256 half.  Barrier roles as in the pair GEMM: full[] and
// tempty[] live in the leader, empty[] and tfull[] in both CTAs (multicast commit).
// Used for forward and stride-1 dgrad when C % 32 == 0 and there are more than 128 output channels.
// ---------------------------------------------------------------------------------------------
constexpr int P2_BN = 256;
constexpr int P2_B_STAGE_BYTES = (P2_BN / 2) * BK * 4;
constexpr int P2_STAGE_BYTES = A_STAGE_BYTES + P2_B_STAGE_BYTES;
constexpr int P2_STAGES = 6;
constexpr int P2_STAT_BYTES = 4 * 2 * P2_BN * 4;
constexpr int P2_SMEM_BYTES = STORE_STAGING_BYTES + P2_STAT_BYTES + P2_STAGES * P2_STAGE_BYTES + 1024 + 256;

// Forward pair kernel, written for tiles of BN = 64 / 128 / 256 output channels; only BN = 256 is
// dispatched (see run_forward for the measurement that keeps narrow tiles on the one-CTA kernel).
template <int BN>
struct PairCfg {
  static constexpr int B_STAGE_BYTES = (BN / 2) * BK * 4;       // this CTA's half of the filter rows
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = BN == 256 ? 6 : 8;
  static constexpr int STAT_BYTES = 4 * 2 * BN * 4;
  static constexpr int SMEM_BYTES = STORE_STAGING_BYTES + STAT_BYTES + STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;    // two accumulators; 128, 256 or 512 columns
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
conv_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmi,
                     const __grid_constant__ CUtensorMap tmo, const ConvParams p) {
  using PC = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_stg = smem;
  float* smem_stat = reinterpret_cast<float*>(smem + STORE_STAGING_BYTES);
  uint8_t* smem_a = smem + STORE_STAGING_BYTES + PC::STAT_BYTES;
  uint8_t* smem_b = smem_a + PC::STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_a + PC::STAGES * PC::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + PC::STAGES;
  uint64_t* tfull = bars + 2 * PC::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PC::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm);
    tma_prefetch_desc(&tmi);
    tma_prefetch_desc(&tmo);
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, PC::TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ptm = (p.M + 255) / 256, ptn = (p.NC + BN - 1) / BN;
  const int items = ptm * ptn;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const int cpb = p.C >> 5;
      for (int item = pair; item < items && ok; item += npairs) {
        const int m0 = (item / ptn) * 256 + (int)rank * 128;          // this CTA's pixels
        const int n0 = (item % ptn) * BN + (int)rank * (BN / 2);  // this CTA's filter rows
        const int n = m0 / (p.OH * p.OW);
        const int rem = m0 - n * (p.OH * p.OW);
        const int oy = rem / p.OW, ox = rem - oy * p.OW;
        const int bw = ox * p.stride - p.pw, bh = oy * p.stride - p.ph;
        int cb = 0, kh = 0, kw = 0;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % PC::STAGES;
          const uint32_t ph = (it / PC::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x211)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * PC::STAGE_BYTES);
          tma_load_im2col_4d_2sm(smem_a + s * A_STAGE_BYTES, &tmi, &full[s], cb * 32, bw, bh, n, (uint16_t)kw,
                                 (uint16_t)kh);
          tma_load_2d_2sm(smem_b + s * PC::B_STAGE_BYTES, &tm, &full[s], kb * BK, n0);
          if (++cb == cpb) {
            cb = 0;
            if (++kw == p.KW) { kw = 0; ++kh; }
          }
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(256, BN, 0, 0);
      constexpr uint32_t HI = smem_desc_hi(1024);
      constexpr uint32_t KSTEP = (UMMA_K * 4) >> 4;
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), 16);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int item = pair; item < items && ok; item += npairs, ++acc_it) {
        const int acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, 0x212)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % PC::STAGES;
          const uint32_t ph = (it / PC::STAGES) & 1;
          if (!mbar_wait(&full[s], ph, p.status, 0x213)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (PC::B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_tf32_2sm(d_tmem, smem_desc_join(HI, a_lo + k * KSTEP), smem_desc_join(HI, b_lo + k * KSTEP), idesc,
                          (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_2sm(&empty[s], 3);
        }
        if (ok) umma_commit_2sm(&tfull[acc], 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs): TMEM -> smem -> TMA store
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    uint8_t* stg = smem_stg + q * 2048;
    const uint32_t srow = smem_u32(stg) + lane * 64;
    const uint32_t sx = (uint32_t)(lane >> 1) & 3;
    float* my_stat = smem_stat + q * 2 * BN;
    if (p.stats)
      for (int i = lane; i < 2 * BN; i += 32) my_stat[i] = 0.f;
    for (int item = pair; item < items && ok; item += npairs, ++acc_it) {
      const int m0 = (item / ptn) * 256 + (int)rank * 128;
      const int n0 = (item % ptn) * BN;
      const int acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, p.status, 0x214)) { ok = false; break; }
      tc_fence_after();
      const int row0 = m0 + q * 32;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tmem_base + acc * BN + ((uint32_t)(q * 32) << 16) + c0, v);
        tmem_ld_wait();
        const int col = n0 + c0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (lane == 0) bulk_wait_read();
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = half * 16 + c * 4;
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(srow + (((uint32_t)c ^ sx) << 4)),
                         "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                         : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && row0 < p.M && col + half * 16 < p.NC) {
            tma_store_2d(&tmo, stg, col + half * 16, row0);
            bulk_commit();
          }
          if (p.stats) stat_accumulate(stg, my_stat, c0 + half * 16, lane);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);
    }
    if (lane == 0) bulk_wait_all();
    if (p.stats)                         // the pair count is a multiple of ptn: one column tile per pair
      stat_flush(p, smem_stat, BN, q, lane, (pair / ptn) * 2 + (int)rank, (pair % ptn) * BN);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // nobody leaves or frees TMEM while the partner may still signal or read
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, PC::TMEM_COLS);
  }
}

// CTA-pair wgrad (cta_group::2): the pair computes 256 output channels x 256 (tap, channel) columns
// of dw over a range of pixels.  Each CTA stages its own 128 rows of dy (one chunked box) and its
// own 128 columns of the patch tile (four im2col boxes of 32 pixels x 32 channels); four producer
// threads per CTA share the boxes as in the one-CTA kernel.  Needs O >= 256 (else half of the
// pair's rows would be padding), C % 32 == 0 and the chunked dy view (O % 32 == 0).
__global__ void __launch_bounds__(288, 1)
conv_wgrad_pair_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmi,
                       const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem + STORE_STAGING_BYTES + P2_STAT_BYTES;
  uint8_t* smem_b = smem_a + P2_STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_a + P2_STAGES * P2_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + P2_STAGES;
  uint64_t* tfull = bars + 2 * P2_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

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
    tma_prefetch_desc(&tm);
    tma_prefetch_desc(&tmi);
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, 512);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ptm = (p.M + 255) / 256, ptn = (p.NC + P2_BN - 1) / P2_BN;
  const int tiles = ptm * ptn;
  const int items = tiles * p.splits;
  const int per_split = (p.kblocks + p.splits - 1) / p.splits;

  // producer q of this CTA: chunk q of this CTA's four patch chunks; q == 0 also the dy box and, in the
  // leader, the byte count of both CTAs' boxes
  auto producer = [&](int q) {
    uint32_t it = 0;
    bool ok = true;
    for (int item = pair; item < items && ok; item += npairs) {
      const int tile = item % tiles, split = item / tiles;
      const int m0 = (tile / ptn) * 256 + (int)rank * 128;     // this CTA's rows (output channels)
      const int nt0 = (tile % ptn) * P2_BN;                    // first column of the pair's tile
      const int col = nt0 + ((int)rank * 4 + q) * 32;          // first column of this producer's chunk
      const bool cvalid = col < p.NC;
      const int tap = col / p.C, c0 = col - tap * p.C;
      const int kh = tap / p.KW, kw = tap - kh * p.KW;
      int nv = (p.NC - nt0 + 31) / 32;
      if (nv > 8) nv = 8;
      const uint32_t tx = 2 * A_STAGE_BYTES + nv * (BK * 128);
      const int kb0 = split * per_split, kb1 = min(p.kblocks, kb0 + per_split);
      const int pix0 = kb0 * BK;
      int n = pix0 / (p.OH * p.OW);
      const int rem = pix0 - n * (p.OH * p.OW);
      int oy = rem / p.OW, ox = rem - oy * p.OW;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % P2_STAGES;
        const uint32_t ph = (it / P2_STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, p.status, 0x221 + q)) { ok = false; break; }
        if (q == 0) {
          if (rank == 0) mbar_expect_tx(&full[s], tx);
          tma_load_3d_2sm(smem_a + s * A_STAGE_BYTES, &tm, &full[s], 0, kb * BK, m0 >> 5);
        }
        if (cvalid)
          tma_load_im2col_4d_2sm(smem_b + s * P2_B_STAGE_BYTES + q * (BK * 128), &tmi, &full[s], c0,
                                 ox * p.stride - p.pw, oy * p.stride - p.ph, n, (uint16_t)kw, (uint16_t)kh);
        ox += BK;
        while (ox >= p.OW) { ox -= p.OW; ++oy; }
        while (oy >= p.OH) { oy -= p.OH; ++n; }
      }
    }
    if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
  };

  if (warp == 0) {
    if (lane == 0) producer(0);
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(256, P2_BN, 1, 1);
      constexpr uint32_t HI = smem_desc_hi(512, LAYOUT_SW128_BASE32B);
      constexpr uint32_t KSTEP = 1024 >> 4;
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), BK * 128);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), BK * 128);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int item = pair; item < items && ok; item += npairs, ++acc_it) {
        const int split = item / tiles;
        const int kb0 = split * per_split, kb1 = min(p.kblocks, kb0 + per_split);
        const int acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, 0x225)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P2_BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % P2_STAGES;
          const uint32_t ph = (it / P2_STAGES) & 1;
          if (!mbar_wait(&full[s], ph, p.status, 0x226)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (P2_B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_tf32_2sm(d_tmem, smem_desc_join(HI, a_lo + k * KSTEP), smem_desc_join(HI, b_lo + k * KSTEP), idesc,
                          (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit_2sm(&empty[s], 3);
        }
        if (ok) umma_commit_2sm(&tfull[acc], 3);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int item = pair; item < items && ok; item += npairs, ++acc_it) {
      const int tile = item % tiles, split = item / tiles;
      const int m0 = (tile / ptn) * 256 + (int)rank * 128;
      const int n0 = (tile % ptn) * P2_BN;
      const int kb0 = split * per_split, kb1 = min(p.kblocks, kb0 + per_split);
      const bool has_k = kb0 < kb1;
      const int acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, p.status, 0x227)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      float* crow = p.splits > 1 ? p.ws + ((long long)split * p.M + row) * p.ldc : p.out + (long long)row * p.ldc;
#pragma unroll 1
      for (int c0 = 0; c0 < P2_BN; c0 += 32) {
        float v[32];
        if (has_k) {
          tmem_ld_32x32(tmem_base + acc * P2_BN + ((uint32_t)(q * 32) << 16) + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        const int col = n0 + c0;
        if (row < p.M && col < p.NC) {     // NC is a multiple of 32 here and ldc * 4 of 16: whole chunks, aligned
          float* dst = crow + col;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);
    }
  } else {
    if (lane == 0) producer(warp - 5);      // warps 6, 7, 8: patch chunks 1, 2, 3
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

// ---- few-channel stems (RGB) through the TMA kernels --------------------------------------------
// A stride-1 "same" convolution over x[N,H,W,4] (3 real channels) has K = 9 * 4: far too short for
// a 32-wide k-block.  Reading the same memory as x'[N,H,W/8,32] (eight pixels of a row = one packed
// pixel with 32 channels) and y[N,H,W,O] as y'[N,H,W/8,8*O] turns it into an ordinary 3-wide
// convolution with 32 input and 8*O output channels whose filters are mostly zero:
//   w'[(po, o)][kh][dx + 1][(pi, c)] = w[o][kh][kw][c]  with  kw = 8 * dx + pi - po + pw,  if 0 <= kw < KW.
// Eight times the arithmetic, but on the tensor cores at full rate instead of on the gather path.
__global__ void stem_pack_filters(const float* __restrict__ w, long long so, long long sc, long long sh,
                                  long long sw, float* __restrict__ out, int O, int C, int KH, int KW, int pw) {
  const long long total = 8ll * O * KH * 3 * 32;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int pc = (int)(i % 32);
    long long r = i / 32;
    const int dxi = (int)(r % 3); r /= 3;
    const int kh = (int)(r % KH); r /= KH;
    const int o = (int)(r % O);
    const int po = (int)(r / O);
    const int pi = pc >> 2, c = pc & 3;
    const int kw = 8 * (dxi - 1) + pi - po + pw;
    float v = 0.f;
    if (c < C && kw >= 0 && kw < KW) v = w[o * so + c * sc + kh * sh + kw * sw];
    out[i] = v;
  }
}

// dw[o][kh][kw][c] = sum of the packed gradient entries that alias this filter tap
__global__ void stem_unpack_filter_grads(const float* __restrict__ gp, float* __restrict__ dw, long long so,
                                         long long sc, long long sh, long long sw, int O, int C, int KH, int KW,
                                         int pw) {
  const int total = O * KH * KW * C;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int c = i % C;
    int r = i / C;
    const int kw = r % KW; r /= KW;
    const int kh = r % KH;
    const int o = r / KH;
    float acc = 0.f;
    for (int po = 0; po < 8; ++po) {
      const int t = kw - pw + po;                 // = 8 * dx + pi
      const int dx = (t >= 0) ? t / 8 : -((7 - t) / 8);
      const int pi = t - 8 * dx;
      if (dx < -1 || dx > 1) continue;
      acc += gp[((((long long)po * O + o) * KH + kh) * 3 + (dx + 1)) * 32 + pi * 4 + c];
    }
    dw[o * so + c * sc + kh * sh + kw * sw] = acc;
  }
}

// Strided dgrad runs as a stride-1 forward convolution over dy with zeros inserted between its
// pixels: up[n][s*i][s*j][:] = dy[n][i][j][:], zero elsewhere (Hup x Wup positions).  The inserted
// zeros cost s*s times the arithmetic of the strided layer, but on the TMA kernels.
__global__ void upsample_zero_insert(const float* __restrict__ dy, float* __restrict__ up, int N, int OH, int OW,
                                     int O, int Hup, int Wup, int stride) {
  const int O4 = O >> 2;
  const long long total = (long long)N * Hup * Wup * O4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % O4) * 4;
    long long r = i / O4;
    const int xx = (int)(r % Wup); r /= Wup;
    const int yy = (int)(r % Hup);
    const int n = (int)(r / Hup);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const int iy = yy / stride, ix = xx / stride;
    if (iy * stride == yy && ix * stride == xx && iy < OH && ix < OW)
      v = *reinterpret_cast<const float4*>(dy + (((long long)n * OH + iy) * OW + ix) * O + c);
    *reinterpret_cast<float4*>(up + i * 4) = v;
  }
}

// Stride-2 dgrad without inserted zeros.  dx[2i + a] (a = 0, 1 per axis) only receives the filter taps
// kh = 2t + r with r = (a + pad) & 1, and with q = (a + pad - r) / 2
//     dx_a[i] = sum_t dy[i + q - t] * w[2t + r]
// which is the data gradient of a STRIDE-1 convolution with the sub-filter w[2t + r] (T taps) and padding q.  So
// each of the four (row parity, column parity) classes is one stride-1 forward launch over dy with the class's
// flipped, transposed sub-filter; the four dense results are then interleaved into dx by one kernel.  The launch
// pads dy by T - 1 - q at the leading edge and by R - OH + q at the trailing edge (R = ceil((H - a) / 2) rows of
// the class; the two differ, and the trailing one may be negative), so it produces exactly R rows.
// 3x3 / pad 1: 1 + 2 taps per axis, 9 tap-positions per 2x2 block of dx against 36 on the zero-inserted
// gradient; 1x1 / pad 0: 1 against 4.
struct ParityAxis {
  int r, T, q, R, pad_lead, pad_trail;
  bool empty;            // no tap falls on this parity: the class is zero
};

bool parity_axis(int H, int OH, int K, int pad, int a, ParityAxis* d) {
  d->r = (a + pad) & 1;
  d->T = K > d->r ? (K - d->r + 1) / 2 : 0;
  d->q = (a + pad - d->r) / 2;
  d->R = H > a ? (H - a + 1) / 2 : 0;
  d->empty = d->T == 0;
  d->pad_lead = d->T - 1 - d->q;
  d->pad_trail = d->R - OH + d->q;
  return d->empty || d->R == 0 || (d->pad_lead >= 0 && OH + d->pad_lead + d->pad_trail >= d->T);
}

// out[c][Ta-1-ta][Tb-1-tb][o] = w[o][2ta + ra][2tb + rb][c]: the class's sub-filter, flipped and transposed.
__global__ void parity_filters(const float* __restrict__ w, float* __restrict__ out, int O, int C, int KH, int KW,
                               int ra, int Ta, int rb, int Tb) {
  __shared__ float tile[32][33];
  const int ta = blockIdx.z / Tb, tb = blockIdx.z - ta * Tb;
  const int ftap = (Ta - 1 - ta) * Tb + (Tb - 1 - tb);
  const int tap = (2 * ta + ra) * KW + (2 * tb + rb);
  const int taps = KH * KW, subtaps = Ta * Tb;
  const int c0 = blockIdx.x * 32, o0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int o = o0 + r, c = c0 + threadIdx.x;
    tile[r][threadIdx.x] = (o < O && c < C) ? w[((long long)o * taps + tap) * C + c] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r, o = o0 + threadIdx.x;
    if (c < C && o < O) out[((long long)c * subtaps + ftap) * O + o] = tile[threadIdx.x][r];
  }
}

// dx[n][y][x][:] = part[(y & 1) * 2 + (x & 1)][n][y >> 1][x >> 1][:] (a null part is a class of zeros).  One pass
// over dx with contiguous 16-byte stores; C % 4 == 0.
struct ParityParts {
  const float* part[4];
  int R[4][2];           // rows, columns of each class
};

__global__ void parity_interleave(const ParityParts pp, float* __restrict__ dx, int N, int H, int W, int C) {
  const int C4 = C >> 2;
  const long long total = (long long)N * H * W * C4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C4) * 4;
    long long r = i / C4;
    const int x = (int)(r % W); r /= W;
    const int y = (int)(r % H);
    const int n = (int)(r / H);
    const int k = (y & 1) * 2 + (x & 1);
    const float* src = pp.part[k];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (src)
      v = *reinterpret_cast<const float4*>(src + (((long long)n * pp.R[k][0] + (y >> 1)) * pp.R[k][1] + (x >> 1)) * C + c);
    *reinterpret_cast<float4*>(dx + i * 4) = v;
  }
}

__global__ void conv_splitk_reduce(const float* __restrict__ ws, float* __restrict__ out, int splits,
                                   long long per_split, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < per_split;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[s * per_split + i];
    out[i] = accumulate ? out[i] + acc : acc;
  }
}

// Filters for stride-1 dgrad run through the forward kernel: out[c][KH-1-kh][KW-1-kw][o] = w[o][kh][kw][c].
// One 32x32 tile of the (o, c) plane of one tap per block, transposed through shared memory.
__global__ void flip_transpose_filters(const float* __restrict__ w, float* __restrict__ out, int O, int C, int KH,
                                       int KW) {
  __shared__ float tile[32][33];
  const int tap = blockIdx.z, kh = tap / KW, kw = tap - kh * KW;
  const int ftap = (KH - 1 - kh) * KW + (KW - 1 - kw);
  const int taps = KH * KW;
  const int c0 = blockIdx.x * 32, o0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int o = o0 + r, c = c0 + threadIdx.x;
    tile[r][threadIdx.x] = (o < O && c < C) ? w[((long long)o * taps + tap) * C + c] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r, o = o0 + threadIdx.x;
    if (c < C && o < O) out[((long long)c * taps + ftap) * O + o] = tile[threadIdx.x][r];
  }
}

// Library-owned scratch (split-K partial sums, transposed filters, zero-inserted gradients): one buffer
// per (stream, slot), so that convolutions running concurrently on different streams never share one.
float* get_ws(cudaStream_t st, int slot, size_t bytes, size_t floor_bytes) {
  return static_cast<float*>(tsb_scratch::get(st, tsb_scratch::CONV_SPLITK + slot, bytes, floor_bytes));
}

// TSB_CONV_DGRAD_PARITY=0 selects the zero-insertion path for stride-2 data gradients (for comparison).
bool dgrad_parity_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TSB_CONV_DGRAD_PARITY");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int MODE, int BN, bool IM2COL>
int launch(const CUtensorMap& tm, const CUtensorMap& tmi, const CUtensorMap& tmo, const ConvParams& p,
           cudaStream_t st) {
  using C = Cfg<BN, IM2COL>;
  auto kern = conv_tf32_kernel<MODE, BN, IM2COL>;
  constexpr int threads = IM2COL ? (MODE == 2 ? 288 : 192) : NUM_THREADS;   // wgrad: three extra producer warps
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return TSB_ERR_LAUNCH | ((int)cudaGetLastError() << 8);
    attr_set = true;
  }
  const long long items = (long long)p.tiles_m * p.tiles_n * p.taps * p.splits;
  const long long slots = (long long)sm_count() * C::OCC;
  int grid = (int)(items < slots ? items : slots);
  if (p.stats && grid > p.tiles_n) grid -= grid % p.tiles_n;    // every CTA then sees one column tile only
#ifdef TSB_CONV_PROF
  static unsigned long long* prof = nullptr;
  if (!prof) cudaMalloc(reinterpret_cast<void**>(&prof), 16 * sizeof(unsigned long long));
  cudaMemsetAsync(prof, 0, 16 * sizeof(unsigned long long), st);
  ConvParams pp = p;
  pp.prof = prof;
  kern<<<grid, threads, C::SMEM_BYTES, st>>>(tm, tmi, tmo, pp);
  unsigned long long h[16];
  cudaMemcpyAsync(h, prof, sizeof(h), cudaMemcpyDeviceToHost, st);
  cudaStreamSynchronize(st);
  const double kbs = (double)items / grid * ((p.kblocks + p.splits - 1) / p.splits);   // k-blocks per CTA
  fprintf(stderr,
          "[conv prof] mode %d bn %d im2col %d grid %d kblocks/cta %.0f | cycles per k-block: mma total %.0f (wait "
          "full %.0f, wait tmem %.0f, issue %.0f = 4 mma %.0f + commit %.0f + rest) | tma total %.0f (wait empty %.0f) | gather total %.0f (wait empty "
          "%.0f) | epilogue total %.0f (wait tmem-full %.0f)\n",
          MODE, BN, (int)IM2COL, grid, kbs, h[3] / kbs / grid, h[0] / kbs / grid, h[1] / kbs / grid,
          h[2] / kbs / grid, h[13] / kbs / grid, h[14] / kbs / grid, h[5] / kbs / grid, h[4] / kbs / grid, h[9] / kbs / grid, h[6] / kbs / grid,
          h[12] / kbs / grid, h[11] / kbs / grid);
#else
  kern<<<grid, threads, C::SMEM_BYTES, st>>>(tm, tmi, tmo, p);
#endif
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

template <int MODE, bool IM2COL>
int launch_bn(int bn, const CUtensorMap& tm, const CUtensorMap& tmi, const CUtensorMap& tmo, const ConvParams& p,
              cudaStream_t st) {
  if (bn == 256) return launch<MODE, 256, IM2COL>(tm, tmi, tmo, p, st);
  if (bn == 128) return launch<MODE, 128, IM2COL>(tm, tmi, tmo, p, st);
  return launch<MODE, 64, IM2COL>(tm, tmi, tmo, p, st);
}

template <int BN>
int launch_fwd_pair_bn(const CUtensorMap& tm, const CUtensorMap& tmi, const CUtensorMap& tmo, const ConvParams& p,
                       cudaStream_t st) {
  using PC = PairCfg<BN>;
  auto kern = conv_fwd_pair_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PC::SMEM_BYTES) != cudaSuccess)
      return TSB_ERR_LAUNCH | ((int)cudaGetLastError() << 8);
    attr_set = true;
  }
  const int ptn = (p.NC + BN - 1) / BN;
  const long long items = (long long)((p.M + 255) / 256) * ptn;
  long long pairs = sm_count() / 2;
  if (pairs > items) pairs = items;
  if (p.stats && pairs > ptn) pairs -= pairs % ptn;              // every pair then sees one column tile only
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = PC::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm, tmi, tmo, p);
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

int launch_fwd_pair(int bn, const CUtensorMap& tm, const CUtensorMap& tmi, const CUtensorMap& tmo,
                    const ConvParams& p, cudaStream_t st) {
  if (bn == 256) return launch_fwd_pair_bn<256>(tm, tmi, tmo, p, st);
  if (bn == 128) return launch_fwd_pair_bn<128>(tm, tmi, tmo, p, st);
  return launch_fwd_pair_bn<64>(tm, tmi, tmo, p, st);
}

int launch_wgrad_pair(const CUtensorMap& tm, const CUtensorMap& tmi, const ConvParams& p, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(conv_wgrad_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P2_SMEM_BYTES) !=
        cudaSuccess)
      return TSB_ERR_LAUNCH | ((int)cudaGetLastError() << 8);
    attr_set = true;
  }
  const long long items = (long long)((p.M + 255) / 256) * ((p.NC + P2_BN - 1) / P2_BN) * p.splits;
  long long pairs = sm_count() / 2;
  if (pairs > items) pairs = items;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(288);
  cfg.dynamicSmemBytes = P2_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, conv_wgrad_pair_kernel, tm, tmi, p);
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

ConvParams base_params(int N, int C, int H, int W, int O, int KH, int KW, int OH, int OW, int ph, int pw,
                       int stride) {
  ConvParams p;
  p.N = N; p.C = C; p.H = H; p.W = W; p.O = O; p.KH = KH; p.KW = KW; p.OH = OH; p.OW = OW;
  p.ph = ph; p.pw = pw; p.stride = stride;
  p.src = nullptr; p.out = nullptr; p.ws = nullptr; p.accumulate = 0; p.splits = 1; p.taps = 1;
  p.K = KH * KW * C; p.ocb = (O + 31) / 32; p.status = nullptr; p.prof = nullptr; p.a3d = 0; p.tma_store = 0; p.stats = nullptr; p.stats_plane = 0;
  p.M = 0; p.NC = 0; p.kblocks = 0; p.tiles_m = 0; p.tiles_n = 0; p.ldc = 0;
  return p;
}

// im2col-mode map of the activation `a`[N,H,W,C] for a KHxKW window with this padding and stride.
// Returns TSB_ERR_UNSUPPORTED when the shape is outside what the TMA path handles (the caller
// then gathers with cp.async instead).
// ph / pw pad the top / left edge, ph_end / pw_end the bottom / right edge (they may differ, and the end padding
// may be negative: trailing rows of `a` that no window reaches).
int im2col_map(CUtensorMap* out, const float* a, int N, int C, int H, int W, int KH, int KW, int OH, int OW, int ph,
               int pw, int stride, int pixels, bool atom32, int ph_end, int pw_end) {
  if (C % 32) return TSB_ERR_UNSUPPORTED;
  if (KH > 255 || KW > 255) return TSB_ERR_UNSUPPORTED;
  if (H + ph + ph_end < KH || W + pw + pw_end < KW) return TSB_ERR_UNSUPPORTED;
  if ((H + ph + ph_end - KH) / stride + 1 != OH || (W + pw + pw_end - KW) / stride + 1 != OW)
    return TSB_ERR_UNSUPPORTED;
  const int lower[2] = {-pw, -ph};
  const int upper[2] = {pw_end - (KW - 1), ph_end - (KH - 1)};
  return tsb_host::make_tmap_im2col_f32(out, a, C, W, H, N, lower, upper, 32, pixels, stride, stride, atom32);
}

// out[N,OH,OW,O] = conv(src[N,H,W,C], wts[O,KH,KW,C]).  Serves forward, and stride-1 dgrad with
// flipped and transposed filters.
// stats / stats_plane / max_chunks / chunks_out (optional): also leave per-CTA column sums and sums of
// squares of the output in `stats` ([chunks][O] in each of two planes `stats_plane` floats apart) and
// report the number of chunks; 0 chunks = statistics not produced (the caller computes them itself).
int run_forward(const float* src, const float* wts, float* out, int N, int C, int H, int W, int O, int KH, int KW,
                int OH, int OW, int ph, int pw, int stride, cudaStream_t st, float* stats = nullptr,
                long long stats_plane = 0, int max_chunks = 0, int* chunks_out = nullptr, int ph_end = INT_MIN,
                int pw_end = INT_MIN) {
  if (chunks_out) *chunks_out = 0;
  if (ph_end == INT_MIN) ph_end = ph;      // symmetric padding unless the caller says otherwise
  if (pw_end == INT_MIN) pw_end = pw;
  ConvParams p = base_params(N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride);
  p.status = tsb_host::status_word(st);
  if (!p.status) return TSB_ERR_LAUNCH;
  p.src = src; p.out = out; p.M = N * OH * OW; p.NC = O; p.ldc = O;
  p.kblocks = (p.K + BK - 1) / BK;
  const int bn = O > 128 ? 256 : (O > 64 ? 128 : 64);
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.NC + bn - 1) / bn;
  CUtensorMap tm, tmi;
  uint64_t d[2] = {(uint64_t)p.K, (uint64_t)O}, s[1] = {(uint64_t)p.K * 4};
  uint32_t bx[2] = {BK, (uint32_t)bn};
  int rc = tsb_host::make_tmap_f32(&tm, wts, 2, d, s, bx, false);
  if (rc) return rc;
  // output [M][O] leaves through TMA stores of 32 rows x 16 columns (64-byte rows, 64B swizzle)
  CUtensorMap tmo;
  {
    uint64_t od[2] = {(uint64_t)O, (uint64_t)p.M}, os[1] = {(uint64_t)O * 4};
    uint32_t ob[2] = {16, 32};
    rc = tsb_host::make_tmap_f32_swz(&tmo, out, 2, od, os, ob, 2);
    if (rc) return rc;
    p.tma_store = 1;
  }
  rc = im2col_map(&tmi, src, N, C, H, W, KH, KW, OH, OW, ph, pw, stride, BM, false, ph_end, pw_end);
  if (rc == TSB_OK) {
    const char* e = getenv("TSB_CONV_PAIR");              // "0" selects the one-CTA tiles everywhere
    const int ptn = (p.NC + bn - 1) / bn;
    const long long pair_items = (long long)((p.M + 255) / 256) * ptn;
    // narrow tiles measured slower on pairs (one CTA per SM, one issuing thread per two SMs) than on the
    // one-CTA kernel with two CTAs per SM: 64 -> 64 channels at 224x224, batch 64: 0.90 ms against 0.61 ms
    if (!(e && e[0] == '0') && bn == 256 && pair_items * 4 >= sm_count()) {
      CUtensorMap tmh;          // filters, bn / 2 rows per CTA
      uint32_t hb[2] = {BK, (uint32_t)bn / 2};
      rc = tsb_host::make_tmap_f32(&tmh, wts, 2, d, s, hb, false);
      if (rc) return rc;
      if (stats) {              // same grid arithmetic as launch_fwd_pair_bn
        long long pairs = sm_count() / 2;
        if (pairs > pair_items) pairs = pair_items;
        if (pairs > ptn) pairs -= pairs % ptn;
        const int chunks = (int)(2 * pairs / ptn);
        if (pairs % ptn == 0 && chunks <= max_chunks) {
          p.stats = stats; p.stats_plane = stats_plane;
          if (chunks_out) *chunks_out = chunks;
        }
      }
      return launch_fwd_pair(bn, tmh, tmi, tmo, p, st);
    }
    if (stats) {                // same grid arithmetic as launch<>
      const long long items = (long long)p.tiles_m * p.tiles_n;
      const long long slots = (long long)sm_count() * (bn <= 128 ? 2 : 1);
      int grid = (int)(items < slots ? items : slots);
      if (grid > p.tiles_n) grid -= grid % p.tiles_n;
      const int chunks = grid / p.tiles_n;
      if (grid % p.tiles_n == 0 && chunks <= max_chunks) {
        p.stats = stats; p.stats_plane = stats_plane;
        if (chunks_out) *chunks_out = chunks;
      }
    }
    return launch_bn<0, true>(bn, tm, tmi, tmo, p, st);
  }
  if (rc != TSB_ERR_UNSUPPORTED) return rc;
  return launch_bn<0, false>(bn, tm, tm, tmo, p, st);
}

// dx[N,H,W,C] = stride-2 dgrad(dy[N,OH,OW,O], w[O,KH,KW,C]) by parity classes (see parity_filters).
// Returns TSB_ERR_UNSUPPORTED when a class cannot be written as a stride-1 launch.
int run_dgrad_parity(float* dx, const float* w, const float* dy, int N, int C, int H, int W, int O, int KH, int KW,
                     int OH, int OW, int ph, int pw, cudaStream_t st) {
  ParityAxis ax[2], bx[2];
  for (int a = 0; a < 2; ++a) {
    if (!parity_axis(H, OH, KH, ph, a, &ax[a]) || !parity_axis(W, OW, KW, pw, a, &bx[a])) return TSB_ERR_UNSUPPORTED;
  }
  size_t wmax = 0, ptotal = 0, poff[4] = {0, 0, 0, 0};
  bool live[4];
  for (int a = 0; a < 2; ++a)
    for (int b = 0; b < 2; ++b) {
      const int k = a * 2 + b;
      live[k] = !(ax[a].empty || bx[b].empty || ax[a].R == 0 || bx[b].R == 0);
      if (!live[k]) continue;
      const size_t wb = (size_t)C * ax[a].T * bx[b].T * O * sizeof(float);
      if (wb > wmax) wmax = wb;
      poff[k] = ptotal;
      ptotal += ((size_t)N * ax[a].R * bx[b].R * C * sizeof(float) + 255) & ~size_t(255);
    }
  if (ptotal > (size_t(4) << 30)) return TSB_ERR_UNSUPPORTED;
  // every class has its own filter buffer: the four launches are queued back to back
  float* wt = wmax ? get_ws(st, 1, 4 * wmax, size_t(16) << 20) : nullptr;
  float* parts = ptotal ? get_ws(st, 2, ptotal, size_t(64) << 20) : nullptr;
  if ((wmax && !wt) || (ptotal && !parts)) return TSB_ERR_OOM;
  ParityParts pp;
  for (int a = 0; a < 2; ++a)
    for (int b = 0; b < 2; ++b) {
      const int k = a * 2 + b;
      const ParityAxis &A = ax[a], &B = bx[b];
      pp.part[k] = nullptr;
      pp.R[k][0] = A.R; pp.R[k][1] = B.R;
      if (!live[k]) continue;
      float* wk = wt + (size_t)k * (wmax / sizeof(float));
      float* part = reinterpret_cast<float*>(reinterpret_cast<char*>(parts) + poff[k]);
      dim3 grid((C + 31) / 32, (O + 31) / 32, A.T * B.T);
      parity_filters<<<grid, dim3(32, 8), 0, st>>>(w, wk, O, C, KH, KW, A.r, A.T, B.r, B.T);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
      const int rc = run_forward(dy, wk, part, N, O, OH, OW, C, A.T, B.T, A.R, B.R, A.pad_lead, B.pad_lead, 1, st,
                                 nullptr, 0, 0, nullptr, A.pad_trail, B.pad_trail);
      if (rc) return rc;
      pp.part[k] = part;
    }
  const long long work = (long long)N * H * W * (C / 4);
  long long blocks = (work + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  parity_interleave<<<(unsigned)blocks, 256, 0, st>>>(pp, dx, N, H, W, C);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
  return TSB_OK;
}

}  // namespace

extern "C" {

// Geometry of one parity class of a stride-2 data gradient along one axis (host arithmetic only; see
// parity_filters).  out = {r, T, q, R, leading pad, trailing pad, empty}; returns 1 if the class can run as a stride-1 launch.
int tsb_conv_parity_axis(int H, int OH, int K, int pad, int a, int* out) {
  ParityAxis d;
  const bool ok = parity_axis(H, OH, K, pad, a, &d);
  if (out) {
    out[0] = d.r; out[1] = d.T; out[2] = d.q; out[3] = d.R; out[4] = d.pad_lead; out[5] = d.pad_trail;
    out[6] = d.empty ? 1 : 0;
  }
  return ok ? 1 : 0;
}

// kind 0: y = conv(x, w);  1: x(dx) = dgrad(y(dy), w);  2: w(dw) = wgrad(x, y(dy)).
// x[N,H,W,C], w[O,KH,KW,C], y[N,OH,OW,O] dense channels-last fp32; C % 4 == 0 and O % 4 == 0.
int tsb_conv2d(int kind, float* x, float* w, float* y, int N, int C, int H, int W, int O, int KH, int KW, int OH,
               int OW, int ph, int pw, int stride, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kind < 0 || kind > 2 || N <= 0 || stride <= 0) return TSB_ERR_ARG;
  if ((C % 4) || (O % 4)) return TSB_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return TSB_ERR_UNSUPPORTED;
  if ((long long)N * OH * OW >= (1ll << 31) || (long long)N * H * W >= (1ll << 31)) return TSB_ERR_UNSUPPORTED;
  int rc;
  if (kind == 0) {
    rc = run_forward(x, w, y, N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride, st);
  } else if (kind == 1 && stride == 1 && (O % 32) == 0 && ph <= KH - 1 && pw <= KW - 1) {
    // stride-1 dgrad = forward convolution of dy with the flipped, transposed filters
    const size_t wbytes = (size_t)C * KH * KW * O * sizeof(float);
    float* wt = get_ws(st, 1, wbytes, size_t(16) << 20);
    if (!wt) return TSB_ERR_OOM;
    dim3 grid((C + 31) / 32, (O + 31) / 32, KH * KW);
    flip_transpose_filters<<<grid, dim3(32, 8), 0, st>>>(w, wt, O, C, KH, KW);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
    rc = run_forward(y, wt, x, N, O, OH, OW, C, KH, KW, H, W, KH - 1 - ph, KW - 1 - pw, 1, st);
  } else if (kind == 1 && stride == 2 && (O % 32) == 0 && ph <= KH - 1 && pw <= KW - 1 && dgrad_parity_enabled() &&
             (rc = run_dgrad_parity(x, w, y, N, C, H, W, O, KH, KW, OH, OW, ph, pw, st)) != TSB_ERR_UNSUPPORTED) {
    // stride-2 dgrad as four stride-1 launches over dy, one per output-pixel parity (rc holds the outcome)
  } else if (kind == 1 && stride > 1 && (O % 32) == 0 && ph <= KH - 1 && pw <= KW - 1 &&
             (long long)N * (H - KH + 1 + 2 * ph) * (W - KW + 1 + 2 * pw) * O * 4 <= (4ll << 30)) {
    // strided dgrad = stride-1 forward convolution of the zero-inserted dy with the flipped, transposed filters
    const int Hup = H - KH + 1 + 2 * ph, Wup = W - KW + 1 + 2 * pw;
    const size_t wbytes = (size_t)C * KH * KW * O * sizeof(float);
    const size_t ubytes = (size_t)N * Hup * Wup * O * sizeof(float);
    float* wt = get_ws(st, 1, wbytes, size_t(16) << 20);
    float* up = get_ws(st, 2, ubytes, size_t(64) << 20);
    if (!wt || !up) return TSB_ERR_OOM;
    dim3 grid((C + 31) / 32, (O + 31) / 32, KH * KW);
    flip_transpose_filters<<<grid, dim3(32, 8), 0, st>>>(w, wt, O, C, KH, KW);
    const long long work = (long long)N * Hup * Wup * (O / 4);
    long long blocks = (work + 255) / 256;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    upsample_zero_insert<<<(unsigned)blocks, 256, 0, st>>>(y, up, N, OH, OW, O, Hup, Wup, stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
    rc = run_forward(up, wt, x, N, O, Hup, Wup, C, KH, KW, H, W, KH - 1 - ph, KW - 1 - pw, 1, st);
  } else if (kind == 1) {
    ConvParams p = base_params(N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride);
    p.status = tsb_host::status_word(st);
    if (!p.status) return TSB_ERR_LAUNCH;
    p.src = y; p.out = x; p.M = N * H * W; p.NC = C; p.ldc = C;
    p.kblocks = KH * KW * p.ocb;
    const int bn = C > 128 ? 256 : (C > 64 ? 128 : 64);
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.NC + bn - 1) / bn;
    CUtensorMap tm;
    uint64_t d[3] = {(uint64_t)C, (uint64_t)KH * KW, (uint64_t)O};
    uint64_t s[2] = {(uint64_t)C * 4, (uint64_t)KH * KW * C * 4};
    uint32_t bx[3] = {32, 1, BK};
    rc = tsb_host::make_tmap_f32(&tm, w, 3, d, s, bx, true);
    if (rc) return rc;
    rc = launch_bn<1, false>(bn, tm, tm, tm, p, st);
  } else {
    ConvParams p = base_params(N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride);
    p.status = tsb_host::status_word(st);
    if (!p.status) return TSB_ERR_LAUNCH;
    const long long mpix = (long long)N * OH * OW;
    p.src = x; p.out = w; p.M = O; p.NC = KH * KW * C; p.ldc = (long long)KH * KW * C;
    p.kblocks = (int)((mpix + BK - 1) / BK);
    const int bn = p.NC > 128 ? 256 : (p.NC > 64 ? 128 : 64);
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.NC + bn - 1) / bn;
    CUtensorMap tm, tmi;
    const bool want_im2col = (C % 32) == 0;
    if (want_im2col && (O % 32) == 0) {
      // chunk-outermost view of dy: one box brings the four 32-channel chunks of a k-block
      uint64_t d[3] = {32, (uint64_t)mpix, (uint64_t)O / 32}, s[2] = {(uint64_t)O * 4, 128};
      uint32_t bx[3] = {32, BK, BM / 32};
      rc = tsb_host::make_tmap_f32(&tm, y, 3, d, s, bx, true);
      p.a3d = 1;
    } else {
      uint64_t d[2] = {(uint64_t)O, (uint64_t)mpix}, s[1] = {(uint64_t)O * 4};
      uint32_t bx[2] = {32, BK};
      rc = tsb_host::make_tmap_f32(&tm, y, 2, d, s, bx, true);
    }
    if (rc) return rc;
    // CTA pairs when there are at least 256 output channels (a pair's 256 rows) and both operands go by TMA
    bool use_pair = false;
    {
      const char* e = getenv("TSB_CONV_PAIR");
      use_pair = !(e && e[0] == '0') && p.a3d && O >= 256 && bn == 256;
    }
    // split the pixel reduction so that the work items fill whole waves of CTAs (or CTA pairs)
    const long long tiles = use_pair ? (long long)((p.M + 255) / 256) * ((p.NC + P2_BN - 1) / P2_BN)
                                     : (long long)p.tiles_m * p.tiles_n * p.taps;
    const int sms = use_pair ? sm_count() / 2 : sm_count();
    int splits = 1;
    double best_eff = 0.0;
    for (int waves = 1; waves <= 4; ++waves) {
      int sp = (int)((long long)waves * sms / tiles);
      if (sp < 1) sp = 1;
      if (sp > p.kblocks / 4) sp = p.kblocks / 4 > 0 ? p.kblocks / 4 : 1;
      if (sp > 64) sp = 64;
      const long long items = tiles * sp;
      const double eff = (double)items / (double)(((items + sms - 1) / sms) * sms);
      // prefer more waves only when they are clearly better balanced (each split costs a partial-sum pass)
      if (eff > best_eff + 0.04) { best_eff = eff; splits = sp; }
    }
    const int per = (p.kblocks + splits - 1) / splits;
    p.splits = (p.kblocks + per - 1) / per;
    if (p.splits > 1) {
      const size_t need = (size_t)p.splits * O * KH * KW * C * sizeof(float);
      p.ws = get_ws(st, 0, need, size_t(128) << 20);
      if (!p.ws) return TSB_ERR_OOM;
    }
    rc = im2col_map(&tmi, x, N, C, H, W, KH, KW, OH, OW, ph, pw, stride, BK, true, ph, pw);
    if (rc == TSB_OK) {
      rc = use_pair ? launch_wgrad_pair(tm, tmi, p, st) : launch_bn<2, true>(bn, tm, tmi, tm, p, st);
    } else if (rc == TSB_ERR_UNSUPPORTED) {
      if (p.a3d) {               // the gather kernel reads dy through the 2-D view
        uint64_t d[2] = {(uint64_t)O, (uint64_t)mpix}, s[1] = {(uint64_t)O * 4};
        uint32_t bx[2] = {32, BK};
        rc = tsb_host::make_tmap_f32(&tm, y, 2, d, s, bx, true);
        if (rc) return rc;
        p.a3d = 0;
      }
      rc = launch_bn<2, false>(bn, tm, tm, tm, p, st);
    }
    if (rc) return rc;
    if (p.splits > 1) {
      const long long per_split = (long long)O * KH * KW * C;
      int blocks = (int)((per_split + 255) / 256);
      if (blocks > sm_count() * 8) blocks = sm_count() * 8;
      conv_splitk_reduce<<<blocks, 256, 0, st>>>(p.ws, p.out, p.splits, per_split, 0);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return TSB_ERR_LAUNCH | ((int)e << 8);
    }
  }
  if (rc) return rc;
  const int late = tsb_host::peek_status();
  return late ? TSB_ERR_TIMEOUT | (late << 8) : TSB_OK;
}

// Forward convolution that also leaves the column statistics of y for a batch norm that follows
// (see run_forward).  *chunks_out == 0 on return means "no statistics": unsupported shape for the
// fused path, or more chunks than the caller's buffer holds.
int tsb_conv2d_fwd_stats(float* x, float* w, float* y, int N, int C, int H, int W, int O, int KH, int KW, int OH,
                         int OW, int ph, int pw, int stride, float* stats, long long stats_plane, int max_chunks,
                         int* chunks_out, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (N <= 0 || stride <= 0 || !chunks_out) return TSB_ERR_ARG;
  *chunks_out = 0;
  if ((C % 4) || (O % 4)) return TSB_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return TSB_ERR_UNSUPPORTED;
  if ((long long)N * OH * OW >= (1ll << 31) || (long long)N * H * W >= (1ll << 31)) return TSB_ERR_UNSUPPORTED;
  int rc = run_forward(x, w, y, N, C, H, W, O, KH, KW, OH, OW, ph, pw, stride, st, stats, stats_plane, max_chunks,
                       chunks_out);
  if (rc) return rc;
  const int late = tsb_host::peek_status();
  return late ? TSB_ERR_TIMEOUT | (late << 8) : TSB_OK;
}

// Packed-stem helpers (see stem_pack_filters).  w / dw are addressed through element strides
// (output channel, input channel, kh, kw) so any filter layout works; the packed array is dense
// [8*O][KH][3][32].
int tsb_stem_pack_filters(const float* w, long long so, long long sc, long long sh, long long sw, float* packed,
                          int O, int C, int KH, int KW, int pw, void* stream) {
  if (C > 4 || KW > 9 || pw > 8 || KW - 1 - pw > 8) return TSB_ERR_UNSUPPORTED;
  const long long total = 8ll * O * KH * 3 * 32;
  stem_pack_filters<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, so, sc, sh, sw, packed, O, C, KH, KW, pw);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

int tsb_stem_unpack_filter_grads(const float* packed, float* dw, long long so, long long sc, long long sh,
                                 long long sw, int O, int C, int KH, int KW, int pw, void* stream) {
  if (C > 4 || KW > 9 || pw > 8 || KW - 1 - pw > 8) return TSB_ERR_UNSUPPORTED;
  const int total = O * KH * KW * C;
  stem_unpack_filter_grads<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      packed, dw, so, sc, sh, sw, O, C, KH, KW, pw);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8));
}

}  // extern "C"
