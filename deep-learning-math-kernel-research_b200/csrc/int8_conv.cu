// INT8 (u8 activations x s8 weights -> s32) direct convolution for sm_100a.
//
// Replaces the reference's elx_int8_conv_direct_1x1_t (src/elx_int8_conv_direct_1x1.cpp:409-480,
// src/elx_int8_conv_direct_1x1_xopt.hpp:20-101), elx_int8_conv_direct_t
// (src/elx_int8_conv_direct.cpp:502-571, src/elx_int8_conv_direct_xopt.hpp:20-110) and the
// micro-kernels under them (src/kernel/elk_u8s8_gemm.hxx:269-406, src/kernel/elk_u8s8_conv.hxx:254-677).
//
// i8_umma_kernel: implicit GEMM  D[pixel][oc] = sum_k A[pixel][k] * B[oc][k]  on tcgen05 tensor
// cores.  One CTA = 2 + I8_EPI_WARPS (8) warps with fixed roles:
//   warp 0      producer: TMA copies global -> shared, STAGES-deep ring, mbarrier complete_tx
//   warp 1      allocates TMEM; lane 0 issues tcgen05.mma (kind::i8, M=128, N=BN, K=32 per
//               instruction) and commits to the ring's "empty" barriers / the accumulator barrier
//   warps 2..   epilogue: tcgen05.ld the s32 accumulators (one pixel per thread), fused
//               scale/shift/sum/ReLU/requantise, 16-byte stores into nChw16c
// Two TMEM accumulator buffers let the epilogue of tile i overlap the MMAs of tile i+1.  The grid
// is persistent: min(#tiles, #SMs) CTAs walk the tile list with stride gridDim.x.
//
// Operand layout in shared memory (both K-major, no swizzle): [K chunk of 16 B][row][16 B], i.e.
// 8 rows x 16 B core matrices; rows of A are output pixels, rows of B are output channels.  The
// nChw16c activation layout already IS that layout: 16 channels of one pixel are 16 contiguous
// bytes and consecutive pixels are consecutive 16-byte groups, so
//   FLAT mode (1x1, stride 1, no padding): a K chunk of a 128-pixel tile is one or two contiguous
//        runs of global memory -> plain bulk copies;
//   BOX mode (KxK, padding, stride 1|2): the tile is a BH x BW rectangle of output pixels and a K
//        chunk is a (16 B, BW, BH) box of the input plane shifted by the filter tap -> one tiled
//        TMA copy per stage, out-of-image taps arrive as zeros from the TMA unit.  Stride 2 is
//        handled by four tensor maps, one per (row, column) parity plane of the input.
// Weights are packed once on the host into exactly the shared-memory image of each
// (oc tile, K stage), so a stage of B is a single contiguous bulk copy.
#include "elb_common.cuh"
#include "umma.cuh"
#include <cstdlib>

namespace elb {

namespace {

constexpr int BM = 128;
#ifndef I8_EPI_WARPS
#define I8_EPI_WARPS 8
#endif
// 2 warps per TMEM lane quarter, interleaved over the 16-channel blocks.  (4 per quarter measured
// slower on the 1x1 benchmark layer, 15.7 vs 13.6 us: the epilogue is bound by the conversion unit,
// two int<->float conversions per output, not by the number of warps.)
constexpr int NUM_EPI_WARPS = I8_EPI_WARPS;
constexpr int EPI_PER_QUARTER = NUM_EPI_WARPS / 4;
constexpr int MAX_PRODUCERS = 4;                                                // warp 0 and the last three warps
constexpr int NUM_THREADS = 64 + NUM_EPI_WARPS * 32 + 32 * (MAX_PRODUCERS - 1);
constexpr int PRODUCER2_WARP = 2 + NUM_EPI_WARPS;
constexpr int MAX_OC_SMEM = 2048;    // per-channel constants cached in shared memory

__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
}

template <int BN, int KC, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = KC * BM * 16;
  static constexpr int B_BYTES = KC * BN * 16;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = RING_BYTES;                       // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int MISC_OFF = BAR_OFF + (2 * STAGES + 4) * 8;  // tmem slot, abort flag
  static constexpr int CONST_OFF = (MISC_OFF + 16 + 15) / 16 * 16; // scale[MAX_OC_SMEM], shift[MAX_OC_SMEM]
  static constexpr int TAP_OFF = CONST_OFF + 2 * MAX_OC_SMEM * 4;  // the copy table (I8ConvParams::tap_tbl)
  static constexpr int TOTAL = TAP_OFF + I8_TAP_TBL_MAX * 4 + 128; // +128: manual alignment slack
};

// optional per-CTA timeline (SM cycle counter), 64 slots per CTA; used by the profiling notes
#define ELB_TRACE(slot) do { if (tracing && (slot) < 64) p.trace[blockIdx.x * 64 + (slot)] = clock64(); } while (0)

// SPEC: 0 = everything decided at run time; 1 / 2 = BOX mode with the copy table, no timeline, rows
// of a box merged (stride 1) / not merged: the long launches, compiled with those flags as
// constants.  The producer and issuer loops are single warps / threads whose every instruction and
// branch costs its latency.  These kernels also issue ALL the MMAs of a last, partly filled K stage:
// the packed weights of the chunks past the end of K are zero, so whatever bytes the unfetched part
// of the slot holds contribute nothing, and the issuer loop needs no per-MMA guard.
template <int BN, int KC, int STAGES, int MODE, int SPEC = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1) i8_umma_kernel(const __grid_constant__ I8ConvParams p) {
  using L = SmemLayout<BN, KC, STAGES>;
  const bool tracing = SPEC != 0 ? false : p.trace != nullptr;
  const bool merged_rows = SPEC == 1 ? true : SPEC == 2 ? false : p.merged_rows != 0;
  const bool use_tbl = SPEC != 0 ? true : p.tap_tbl != nullptr;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
  uint64_t *empty = full + STAGES;
  uint64_t *tfull = empty + STAGES;
  uint64_t *tempty = tfull + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFF + 4);
  float *s_scale = reinterpret_cast<float *>(smem + L::CONST_OFF);
  float *s_shift = s_scale + MAX_OC_SMEM;
  uint32_t *s_tap = reinterpret_cast<uint32_t *>(smem + L::TAP_OFF);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;          // two accumulator buffers (power of two >= 32)
  const int total_tiles = p.m_tiles * p.n_tiles;

  // Set-up in two groups, so that the first copies are on their way while the rest of the CTA is
  // still getting ready (measured on the 1x1 benchmark layer: with one CTA-wide barrier the first
  // copy was issued 4.6-5.0 k cycles into a 22 k-cycle kernel):
  //   producers (warp 0 and the last three warps) only need the barriers: they wait on named
  //   barrier 1 for the MMA warp, which initialises them, and start fetching;
  //   MMA and epilogue warps load the per-channel constants, allocate tensor memory and meet on
  //   named barrier 2.
  const bool is_producer = warp == 0 || warp >= PRODUCER2_WARP;
  if (threadIdx.x == 0) {
    ELB_TRACE(0);
    // the copy engine fetches a tensor map from global memory on first use (a few microseconds cold):
    // start that now
    if (MODE == I8_MODE_BOX)
      for (int i = 0; i < p.stride * p.stride; ++i) tma_prefetch_desc(&p.tmap[i]);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(&tfull[b], 1);
        mbar_init(&tempty[b], NUM_EPI_WARPS);      // one arrival per epilogue warp
      }
      *abort_flag = 0;
      fence_barrier_init();
      fence_proxy_async_smem();
    }
    __syncwarp();
  }
  if (MODE == I8_MODE_BOX && is_producer && use_tbl) {
    const int ptid = (warp == 0 ? 0 : warp - PRODUCER2_WARP + 1) * 32 + lane;
    for (int i = ptid; i < p.tap_n; i += 32 * MAX_PRODUCERS) s_tap[i] = __ldg(p.tap_tbl + i);
  }
  if (is_producer || warp == 1) named_bar_sync(1, 32 * (MAX_PRODUCERS + 1));
  if (!is_producer) {
    for (int i = threadIdx.x - 32; i < p.OCB * V; i += 32 * (1 + NUM_EPI_WARPS)) {
      s_scale[i] = p.scale[i];
      s_shift[i] = p.shift[i];
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before_sync();
    named_bar_sync(2, 32 * (1 + NUM_EPI_WARPS));
    tc_fence_after_sync();
  }
  const uint32_t tmem_base = is_producer ? 0u : *tmem_slot;      // (producers never touch tensor memory)
  if (threadIdx.x == 0) ELB_TRACE(1);
  // Everything above touched only this plan's constants.  The kernel after this one may set itself up
  // now; this one reads its input (and later writes its output) only once the kernel before it is done:
  // the producers wait here, every other role acts on what the producers' copies deliver.
  if (threadIdx.x == 0) griddep_launch_dependents();
  if (is_producer) griddep_wait();
  int fail_code = 0;

  if (warp == 0 || warp >= PRODUCER2_WARP) {
    // ------------------------------------------------------------------ producer(s)
    // BOX mode runs two producer warps that take turns on the passes (two stages each) of the K
    // loop, so that four stages are being issued at any time; see the comment in the loop.
    const uint32_t pw = warp == 0 ? 0u : static_cast<uint32_t>(warp - PRODUCER2_WARP + 1);
    const uint32_t nprod = MODE == I8_MODE_BOX ? static_cast<uint32_t>(p.nprod) : 1u;      // 1, 2 or 4 warps take turns
    uint32_t it = 0, gpass = 0;
    bool ok = pw < nprod;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
      // tile geometry
      int n0 = 0, p0 = 0, rows = BM, oh0 = 0, ow0 = 0;
      if (MODE == I8_MODE_FLAT) {
        const int m0 = mt * BM;
        rows = min(BM, p.M - m0);
        n0 = m0 / p.HW;
        p0 = m0 - n0 * p.HW;
      } else {
        const int per_img = p.tiles_h * p.tiles_w;
        n0 = mt / per_img;
        const int r = mt - n0 * per_img;
        oh0 = (r / p.tiles_w) * p.BH;
        ow0 = (r % p.tiles_w) * p.BW;
      }
      // Every tile walks the K stages in a rotated order (start = tile index mod k_stages): the CTAs
      // of a wave all need the same weight panel, and walking it in lockstep would have them hit the
      // same L2 lines at the same time.  Integer accumulation does not depend on the order.
      const int ks0 = p.rotate_k ? tile % p.k_stages : 0;
      if (MODE == I8_MODE_FLAT) {
        for (int ki = 0; ki < p.k_stages; ++ki, ++it) {
          const int ks = ki + ks0 < p.k_stages ? ki + ks0 : ki + ks0 - p.k_stages;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_warp(&empty[s], ph ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
          uint8_t *a_dst = smem + s * L::STAGE_BYTES;
          uint8_t *b_dst = a_dst + L::A_BYTES;
          const int8_t *b_src = p.wpack + (static_cast<size_t>(nt) * p.k_stages + ks) * L::B_BYTES;
          const int cb0 = ks * KC;
          const int nchunks = min(KC, p.CB - cb0);
          if (lane == 0) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(nchunks * rows * 16 + L::B_BYTES));
          __syncwarp();
          if (lane < nchunks) {
            // rows [0, rows) of the tile = pixels p0.. of image n0, continuing into the next images
            int done = 0, n = n0, pp = p0;
            while (done < rows) {
              const int len = min(rows - done, p.HW - pp);
              const uint8_t *src = p.in + ((static_cast<size_t>(n) * p.CB + cb0 + lane) * p.HW + pp) * 16;
              tma_bulk_g2s(a_dst + lane * (BM * 16) + done * 16, src, static_cast<uint32_t>(len * 16), &full[s]);
              done += len;
              pp = 0;
              ++n;
            }
          } else if (lane == KC) {
            tma_bulk_g2s(b_dst, b_src, L::B_BYTES, &full[s]);
          }
          if (lane == 0 && it < 16) ELB_TRACE(2 + it);
        }
      } else {
        // BOX mode.  Issuing a copy costs its lane a few hundred cycles, copies issued by different
        // lanes of one instruction overlap and different warps issue independently.  A pass serves
        // p.spp pipeline stages: lanes 0..15 one stage, lanes 16..31 (spp = 2) the next; in
        // each group lanes 0..7 fetch the pixels (one tiled copy per box_c channel blocks of one
        // tap: box_c divides CB, so a copy never straddles two taps) and lane 8 the weight panel.
        // Chunks past the end of K are not fetched: their weights are zero, whatever the slot holds.
        const int grp = lane >> 4, gl = lane & 15;
        const int spp = p.spp == 1 ? 1 : 2;          // stages per pass
        // (KC = 16: the host picks box_c >= 2, so at most 8 lanes fetch pixels and lane 15 is free)
        constexpr int B_LANE = KC < 16 ? KC : 15;
        for (int ki0 = 0; ki0 < p.k_stages; ki0 += spp, it += spp, ++gpass) {
          if ((gpass & (nprod - 1u)) != pw) continue;          // another producer warp's pass
          const int ki = ki0 + grp;
          const bool active = grp < spp && ki < p.k_stages;
          const uint32_t my_it = it + grp;
          const int s = my_it % STAGES;
          const uint32_t ph = (my_it / STAGES) & 1u;
          int w_ok = 1;
          if (active && gl == 0) w_ok = mbar_wait(&empty[s], ph ^ 1u, abort_flag) ? 1 : 0;
          if (!__all_sync(0xFFFFFFFFu, w_ok)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
          if (active) {
            const int ks = ki + ks0 < p.k_stages ? ki + ks0 : ki + ks0 - p.k_stages;
            uint8_t *a_dst = smem + s * L::STAGE_BYTES;
            uint8_t *b_dst = a_dst + L::A_BYTES;
            const int8_t *b_src = p.wpack + (static_cast<size_t>(nt) * p.k_stages + ks) * L::B_BYTES;
            const int q0 = ks * KC;
            const int valid = min(KC, p.Q - q0);
            if (gl == 0) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(valid * (BM * 16) + L::B_BYTES));
          }
          __syncwarp();
          if (active) {
            const int ks = ki + ks0 < p.k_stages ? ki + ks0 : ki + ks0 - p.k_stages;
            uint8_t *a_dst = smem + s * L::STAGE_BYTES;
            const int q0 = ks * KC;
            const int valid = min(KC, p.Q - q0);
            if (gl == B_LANE) {
              tma_bulk_g2s(a_dst + L::A_BYTES, p.wpack + (static_cast<size_t>(nt) * p.k_stages + ks) * L::B_BYTES,
                           L::B_BYTES, &full[s]);
            } else if (gl < B_LANE && gl * p.box_c < valid) {
              int cb0, dh, dw, map;
              if (use_tbl) {
                const uint32_t e = s_tap[ks * p.ncopy + gl];
                cb0 = static_cast<int>(e & 0xFFFu);
                dh = static_cast<int>((e >> 12) & 15u) - 8;
                dw = static_cast<int>((e >> 16) & 15u) - 8;
                map = static_cast<int>(e >> 20);
              } else {
                const int q = q0 + gl * p.box_c;
                const int tap = q / p.CB;
                cb0 = q - tap * p.CB;
                // input row = stride*(oh + dh) + parity_h with dh = floor((kh - pad)/stride)
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                const int eh = kh - p.pad_t, ew = kw - p.pad_l;
                dh = (eh >= 0) ? eh / p.stride : -((-eh + p.stride - 1) / p.stride);
                dw = (ew >= 0) ? ew / p.stride : -((-ew + p.stride - 1) / p.stride);
                map = (eh - dh * p.stride) * p.stride + (ew - dw * p.stride);
              }
              const CUtensorMap *tm = &p.tmap[map];
              uint8_t *dst = a_dst + gl * p.box_c * (BM * 16);
              // stride 1: rows of the box are contiguous in memory, so the map describes them as runs of
              // 8-byte elements (2 per pixel) and the TMA unit moves whole rows instead of 16-byte items
              if (merged_rows) tma_tile_4d(dst, tm, (ow0 + dw) * 2, oh0 + dh, cb0, n0, &full[s]);
              else tma_tile_5d(dst, tm, 0, ow0 + dw, oh0 + dh, cb0, n0, &full[s]);
            }
          }
          __syncwarp();
          if (gl == 0 && active && my_it < 16) ELB_TRACE(2 + my_it);
        }
        if (spp == 2 && (p.k_stages & 1)) --it;      // the last pass of an odd K loop served one stage only
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC = umma_idesc(/*c s32*/ 2, /*a u8*/ 0, /*b s8*/ 1, BM, BN);
      uint32_t it = 0, tcount = 0;
      // This loop is ONE thread: every instruction costs its full latency, so the ring slot and its
      // phase are counters and the operand descriptors are a constant upper half plus the stage's
      // shared-memory address (measured: divisions and descriptor construction cost this loop more
      // than issuing the MMAs).
      int s = 0;
      uint32_t ph = 0;
      constexpr uint64_t A_DESC_HI = (static_cast<uint64_t>((BM * 16) >> 4) << 16) | (static_cast<uint64_t>(128 >> 4) << 32) |
                                     (static_cast<uint64_t>(1) << 46);
      constexpr uint64_t B_DESC_HI = (static_cast<uint64_t>((BN * 16) >> 4) << 16) | (static_cast<uint64_t>(128 >> 4) << 32) |
                                     (static_cast<uint64_t>(1) << 46);
      const uint32_t smem_base = smem_u32(smem);
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t b = tcount & 1u, tph = (tcount >> 1) & 1u;
        if (!mbar_wait(&tempty[b], tph ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + b * BN;
        const int ks0 = p.rotate_k ? tile % p.k_stages : 0;      // same rotation as the producer
        int ks = ks0;
        // (Waiting for stage ki + 1 in the middle of stage ki's MMAs, which pays in the fp32 GEMM
        // kernel, measured slower here: 13.2 vs 12.6 us on the 1x1 benchmark layer.)
        for (int ki = 0; ki < p.k_stages; ++ki, ++it) {
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
          tc_fence_after_sync();
          if (it < 16) ELB_TRACE(20 + it);
          const uint32_t a_addr = smem_base + s * L::STAGE_BYTES;
          const uint64_t ad0 = A_DESC_HI | (a_addr >> 4), bd0 = B_DESC_HI | ((a_addr + L::A_BYTES) >> 4);
          // K = 32 bytes = two chunks per instruction; the last stage may hold fewer than KC chunks
          const int pairs = SPEC != 0 ? KC / 2 : (min(KC, p.Q - ks * KC) + 1) >> 1;
#pragma unroll
          for (int k2 = 0; k2 < KC / 2; ++k2) {
            if (SPEC != 0 || k2 < pairs)
              umma_i8(d_tmem, ad0 + ((k2 * 2 * (BM * 16)) >> 4), bd0 + ((k2 * 2 * (BN * 16)) >> 4), IDESC, (ki | k2) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);      // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1u; }
          if (++ks == p.k_stages) ks = 0;
        }
        if (ok) umma_commit(&tfull[b]);  // accumulator complete
        if (tcount == 0) ELB_TRACE(40);
      }
    }
    __syncwarp();
  } else if (warp < PRODUCER2_WARP) {
    // ------------------------------------------------------------------ epilogue (warps 2..)
    const int quarter = warp & 3;                  // TMEM lanes this warp may read: 32*quarter ..
    const int half = (warp - 2) >> 2;              // which of the warps of this quarter
    const int row = quarter * 32 + lane;
    const int elt = p.rq.out_type == OUT_F32 ? 4 : 1;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
      const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
      const uint32_t b = tcount & 1u, tph = (tcount >> 1) & 1u;
      // where does this thread's pixel live?
      bool valid;
      size_t pix_off;      // element offset of channel-block 0 of this pixel, in units of 16 channels
      size_t blk_stride;   // distance between channel blocks, same units
      const float *shift_row = s_shift;      // this pixel's shift vector (border pixels: from the class table)
      if (MODE == I8_MODE_FLAT) {
        const int m = mt * BM + row;
        valid = m < p.M;
        const int n = m / p.HW, pp = m - n * p.HW;
        pix_off = static_cast<size_t>(n) * p.OCB * p.HW + pp;
        blk_stride = p.HW;
      } else {
        const int per_img = p.tiles_h * p.tiles_w;
        const int n = mt / per_img;
        const int r = mt - n * per_img;
        const int oh = (r / p.tiles_w) * p.BH + row / p.BW;
        const int ow = (r % p.tiles_w) * p.BW + row % p.BW;
        valid = oh < p.OH && ow < p.OW;
        pix_off = (static_cast<size_t>(n) * p.OCB * p.OH + oh) * p.OW + ow;
        blk_stride = static_cast<size_t>(p.OH) * p.OW;
        if (p.shift_tbl && valid) {
          const int cls = __ldg(p.hclass + oh) * p.zp_nw + __ldg(p.wclass + ow);
          if (cls != p.zp_full) shift_row = p.shift_tbl + static_cast<size_t>(cls) * (p.OCB * V);
        }
      }
      if (!mbar_wait_warp(&tfull[b], tph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_EPILOGUE; break; }
      tc_fence_after_sync();
      if (tcount == 0 && threadIdx.x == 64) ELB_TRACE(41);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * BN;
      auto emit = [&](int ob, const uint32_t (&r)[16]) {
        const int ocb = nt * (BN / 16) + ob;
        if (valid && ocb < p.OCB) {
          int acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = static_cast<int>(r[i]);
          const size_t off = (pix_off + ocb * blk_stride) * 16;
          if (p.acc_dump) {
            int4 *d = reinterpret_cast<int4 *>(p.acc_dump + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) d[i] = make_int4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
          }
          requant_store16(acc, s_scale + ocb * 16, shift_row + ocb * 16,
                          static_cast<uint8_t *>(p.out) + off * elt, p.rq);
        }
      };
      // This warp owns the 16-channel blocks half, half+P, half+2P, ... (P warps per quarter).
      // Tensor-memory loads are software-pipelined: while one pair of blocks is requantised and
      // stored, the next pair is already on its way.
      constexpr int P = EPI_PER_QUARTER;
      const int nblk = (BN / 16 - half + P - 1) / P;
      const uint32_t w_addr = t_addr + half * 16;      // k-th block of this warp at +16*P*k columns
      uint32_t r0[16], r1[16], r2[16], r3[16];
      if (0 < nblk) tmem_ld16(w_addr, r0);
      if (1 < nblk) tmem_ld16(w_addr + 16 * P, r1);
#pragma unroll 1
      for (int k = 0; k < nblk; k += 4) {
        tmem_ld_wait16(r0);
        tmem_ld_wait16(r1);
        if (k + 2 < nblk) tmem_ld16(w_addr + (k + 2) * 16 * P, r2);
        if (k + 3 < nblk) tmem_ld16(w_addr + (k + 3) * 16 * P, r3);
        emit(half + P * k, r0);
        if (k + 1 < nblk) emit(half + P * (k + 1), r1);
        tmem_ld_wait16(r2);
        tmem_ld_wait16(r3);
        if (k + 4 < nblk) tmem_ld16(w_addr + (k + 4) * 16 * P, r0);
        if (k + 5 < nblk) tmem_ld16(w_addr + (k + 5) * 16 * P, r1);
        if (k + 2 < nblk) emit(half + P * (k + 2), r2);
        if (k + 3 < nblk) emit(half + P * (k + 3), r3);
      }
      tc_fence_before_sync();
      __syncwarp();                             // every lane's tensor-memory loads are done ...
      if (lane == 0) mbar_arrive(&tempty[b]);   // ... before the warp gives the accumulator back
      if (tcount == 0 && threadIdx.x == 64) ELB_TRACE(42);
    }
  }

  // ------------------------------------------------------------------ teardown
  if (fail_code != 0) atomicCAS(p.status, 0, fail_code);
  if (threadIdx.x == 0) ELB_TRACE(43);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// CUDA-core kernel: one thread = one output pixel x 16 output channels, dp4a over the K loop.
// Serves shapes the tensor-core kernels do not take (few channels, odd geometry) and is the
// on-device cross-check of the tcgen05 path in the tests.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) i8_simt_kernel(const __grid_constant__ I8ConvParams p) {
  const long long total = static_cast<long long>(p.N) * p.OH * p.OW;
  const long long m = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int ocb = blockIdx.y;
  if (m >= total) return;
  const int n = static_cast<int>(m / (p.OH * p.OW));
  const int rem = static_cast<int>(m - static_cast<long long>(n) * p.OH * p.OW);
  const int oh = rem / p.OW, ow = rem - oh * p.OW;
  const int ICP = p.CB * 16;
  int acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0;
  for (int kh = 0; kh < p.KH; ++kh) {
    const int ih = oh * p.stride - p.pad_t + kh;
    if (ih < 0 || ih >= p.IH) continue;
    for (int kw = 0; kw < p.KW; ++kw) {
      const int iw = ow * p.stride - p.pad_l + kw;
      if (iw < 0 || iw >= p.IW) continue;
      const int tap = kh * p.KW + kw;
      for (int cb = 0; cb < p.CB; ++cb) {
        const uint4 a = *reinterpret_cast<const uint4 *>(
            p.in + (((static_cast<size_t>(n) * p.CB + cb) * p.IH + ih) * p.IW + iw) * 16);
#pragma unroll
        for (int o = 0; o < 16; ++o) {
          const uint4 w = __ldg(reinterpret_cast<const uint4 *>(
              p.wplain + (static_cast<size_t>(ocb * 16 + o) * p.taps + tap) * ICP + cb * 16));
          int c = acc[o];
          c = dp4a_us(a.x, w.x, c);
          c = dp4a_us(a.y, w.y, c);
          c = dp4a_us(a.z, w.z, c);
          c = dp4a_us(a.w, w.w, c);
          acc[o] = c;
        }
      }
    }
  }
  const size_t off = (((static_cast<size_t>(n) * p.OCB + ocb) * p.OH + oh) * p.OW + ow) * 16;
  if (p.acc_dump) {
#pragma unroll
    for (int i = 0; i < 16; ++i) p.acc_dump[off + i] = acc[i];
  }
  const int elt = p.rq.out_type == OUT_F32 ? 4 : 1;
  const float *shift_row = p.shift;
  if (p.shift_tbl) shift_row = p.shift_tbl + static_cast<size_t>(__ldg(p.hclass + oh) * p.zp_nw + __ldg(p.wclass + ow)) * (p.OCB * V);
  requant_store16(acc, p.scale + ocb * 16, shift_row + ocb * 16, static_cast<uint8_t *>(p.out) + off * elt, p.rq);
}

__global__ void wait_selftest_kernel(int *status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
    const unsigned long long t0 = global_timer_ns();
    bool done = false;
    while (!done) {
      if (mbar_try_wait(&bar, 0)) break;               // never true: nobody arrives
      if (global_timer_ns() - t0 > limit_ns) done = true;
    }
    if (done) *status = ST_WAIT_TIMEOUT_TEST;
    mbar_inval(&bar);
  }
}

template <int BN, int KC, int STAGES, int MODE>
cudaError_t launch_cfg(const I8ConvParams &p, int num_sms, cudaStream_t s, bool attr_only) {
  using L = SmemLayout<BN, KC, STAGES>;
  auto kern = i8_umma_kernel<BN, KC, STAGES, MODE>;
  if (attr_only) {   // once per plan and device, outside any stream capture
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (MODE == I8_MODE_BOX) {
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(i8_umma_kernel<BN, KC, STAGES, MODE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(i8_umma_kernel<BN, KC, STAGES, MODE, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    }
    return e;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  int grid = tiles < num_sms ? tiles : num_sms;
  {
    const int v = tune_env("ELB_MAX_CTAS", grid);
    if (v > 0 && v < grid) grid = v;
  }
  // the kernels compiled for the plain case (see SPEC)
  const bool plain = MODE == I8_MODE_BOX && p.tap_tbl && !p.trace;
  if (MODE == I8_MODE_BOX && plain && p.merged_rows)
    return launch_overlapped(i8_umma_kernel<BN, KC, STAGES, MODE, 1>, dim3(grid), dim3(NUM_THREADS), L::TOTAL, s, p);
  if (MODE == I8_MODE_BOX && plain)
    return launch_overlapped(i8_umma_kernel<BN, KC, STAGES, MODE, 2>, dim3(grid), dim3(NUM_THREADS), L::TOTAL, s, p);
  return launch_overlapped(kern, dim3(grid), dim3(NUM_THREADS), L::TOTAL, s, p);
}

}  // namespace

// Tile configuration.  BN (output channels per tile) in {64, 128, 256}; 8 K-chunks (128 bytes of K)
// per stage; as many stages as fit 227 KB.
I8UmmaConfig i8_umma_config(int ocb, int cb, int taps, int mode) {
  I8UmmaConfig c{};
  c.mode = mode;
  const int ocp = ocb * 16;
  // Per-SM copy ingest (about 50 B/clk) is what bounds these kernels, and the bytes a tile pulls
  // per MAC fall with BN: 256 wherever the channel count allows it (measured on the 1x1 and the
  // 3x3 stride-2 benchmark layers: 13.5 vs 18 us and 39 vs 55 us against BN = 128).
  c.BN = ocp >= 256 ? 256 : ocp >= 128 ? 128 : 64;
  {
    const int v = tune_env("ELB_I8_BN", c.BN);
    if (v == 64 || v == 128 || v == 256) c.BN = v;
  }
  // K chunks (of 16 channels) per stage.  Handing a stage from role to role costs the single-thread
  // role loops about a thousand cycles whatever its size, and the MMAs of a stage of 8 chunks take
  // less than that below 256 output channels: those tiles move 16 chunks per stage (BOX mode needs
  // at most 15 copies per stage for that, i.e. an even number of channel blocks).  A K of 9..16
  // chunks (the 3-channel first layer of an image network) becomes a single stage.
  c.KC = 8;
  // (an odd number of channel blocks is fetched block by block: fine while K has at most 15 of them)
  const bool kc16_ok = c.BN <= 128 && cb * taps > 8 && (mode == I8_MODE_FLAT || cb % 2 == 0 || cb * taps <= 15);
  if (tune_env("ELB_I8_KC", kc16_ok ? 16 : 8) == 16 && kc16_ok) c.KC = 16;
  if (c.KC == 16) {
    c.STAGES = c.BN == 128 ? 3 : 4;
    c.smem_bytes = c.BN == 128 ? SmemLayout<128, 16, 3>::TOTAL : SmemLayout<64, 16, 4>::TOTAL;
    return c;
  }
  c.STAGES = c.BN == 256 ? 4 : c.BN == 128 ? 6 : 8;     // as many as shared memory holds: the ring is latency-bound
  c.smem_bytes = c.BN == 256 ? SmemLayout<256, 8, 4>::TOTAL
               : c.BN == 128 ? SmemLayout<128, 8, 6>::TOTAL : SmemLayout<64, 8, 8>::TOTAL;
  return c;
}

static cudaError_t dispatch_i8_umma(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s,
                                    bool attr_only) {
  if (cfg.KC == 16) {
    if (cfg.mode == I8_MODE_FLAT) {
      if (cfg.BN == 128) return launch_cfg<128, 16, 3, I8_MODE_FLAT>(p, num_sms, s, attr_only);
      return launch_cfg<64, 16, 4, I8_MODE_FLAT>(p, num_sms, s, attr_only);
    }
    if (cfg.BN == 128) return launch_cfg<128, 16, 3, I8_MODE_BOX>(p, num_sms, s, attr_only);
    return launch_cfg<64, 16, 4, I8_MODE_BOX>(p, num_sms, s, attr_only);
  }
  if (cfg.mode == I8_MODE_FLAT) {
    if (cfg.BN == 256) return launch_cfg<256, 8, 4, I8_MODE_FLAT>(p, num_sms, s, attr_only);
    if (cfg.BN == 128) return launch_cfg<128, 8, 6, I8_MODE_FLAT>(p, num_sms, s, attr_only);
    return launch_cfg<64, 8, 8, I8_MODE_FLAT>(p, num_sms, s, attr_only);
  }
  if (cfg.BN == 256) return launch_cfg<256, 8, 4, I8_MODE_BOX>(p, num_sms, s, attr_only);
  if (cfg.BN == 128) return launch_cfg<128, 8, 6, I8_MODE_BOX>(p, num_sms, s, attr_only);
  return launch_cfg<64, 8, 8, I8_MODE_BOX>(p, num_sms, s, attr_only);
}

cudaError_t init_i8_umma(const I8UmmaConfig &cfg) {
  I8ConvParams dummy{};
  return dispatch_i8_umma(dummy, cfg, 1, nullptr, true);
}

cudaError_t launch_i8_umma(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s) {
  if (p.OCB * V > MAX_OC_SMEM) return cudaErrorInvalidValue;
  return dispatch_i8_umma(p, cfg, num_sms, s, false);
}

cudaError_t launch_i8_simt(const I8ConvParams &p, cudaStream_t s) {
  const long long total = static_cast<long long>(p.N) * p.OH * p.OW;
  dim3 grid(static_cast<unsigned>((total + 127) / 128), static_cast<unsigned>(p.OCB));
  i8_simt_kernel<<<grid, 128, 0, s>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_wait_selftest(int *status, unsigned long long limit_ns, cudaStream_t s) {
  wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_ns);
  return cudaGetLastError();
}

}  // namespace elb
