// INT8 direct convolution on PAIRS of SMs: the two-CTA form of the implicit-GEMM kernel in
// int8_conv.cu (same references: src/elx_int8_conv_direct.cpp:502-571,
// src/elx_int8_conv_direct_1x1.cpp:409-480, src/kernel/elk_u8s8_conv.hxx, elk_u8s8_gemm.hxx).
//
// Why: the single-CTA kernel is bound by the bytes an SM has to pull from L2 per tile (measured
// about 34 B/clk per SM with every SM busy), and two thirds of those bytes are the weight panel,
// which every CTA fetches in full.  Here a cluster of two CTAs computes a 256-pixel x BN-channel
// tile with ONE tcgen05.mma.cta_group::2 per K step: each CTA stages its own 128 pixels of A and
// only ITS HALF of the weight rows (BN/2 output channels) in its shared memory, the tensor cores of
// both SMs read both halves, and each SM accumulates its 128 pixels x BN channels in its own tensor
// memory.  Per CTA and stage that is 16 KB + 16 KB instead of 16 KB + 32 KB (BN = 256).
//
// Roles per CTA (10 warps): warp 0 producer (TMA: own pixels, own weight half), warp 1 lane 0: in
// the leader CTA (cluster rank 0) the MMA issuer, in the peer a forwarder that tells the leader
// when the peer's stage has landed (remote mbarrier arrive), warps 2..9 epilogue on the CTA's own
// accumulator.  tcgen05.commit with .multicast::cluster releases a stage / publishes an accumulator
// in both CTAs at once.  No copy in this file uses a cluster-wide (multicast) form.
// Every wait is bounded (umma.cuh); the only unbounded instructions are the cluster barrier at
// start and at teardown, which every thread of both CTAs reaches on every path.
#include "elb_common.cuh"
#include "umma.cuh"
#include <cstdlib>

namespace elb {

namespace {

constexpr int BM = 128;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + NUM_EPI_WARPS * 32;
constexpr int MAX_OC_SMEM = 2048;

template <int BN, int KC, int STAGES>
struct Smem2 {
  static constexpr int A_BYTES = KC * BM * 16;
  static constexpr int B_BYTES = KC * (BN / 2) * 16;               // this CTA's half of the weight rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = RING_BYTES;                       // full[S], empty[S], pfull[S], tfull[2], tempty[2]
  static constexpr int MISC_OFF = BAR_OFF + (3 * STAGES + 4) * 8;  // tmem slot, abort flag
  static constexpr int CONST_OFF = (MISC_OFF + 16 + 15) / 16 * 16;
  static constexpr int TOTAL = CONST_OFF + 2 * MAX_OC_SMEM * 4 + 128;
};

// optional per-CTA timeline (SM cycle counter), 64 slots per CTA; used by the profiling notes
#define ELB_TRACE(slot) do { if (p.trace && (slot) < 64) p.trace[blockIdx.x * 64 + (slot)] = clock64(); } while (0)

template <int BN, int KC, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1) i8_umma2_kernel(const __grid_constant__ I8ConvParams p) {
  using L = Smem2<BN, KC, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
  uint64_t *empty = full + STAGES;
  uint64_t *pfull = empty + STAGES;       // leader only: the peer's stage s has landed
  uint64_t *tfull = pfull + STAGES;
  uint64_t *tempty = tfull + 2;           // leader only: both epilogues are done with accumulator b
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFF + 4);
  float *s_scale = reinterpret_cast<float *>(smem + L::CONST_OFF);
  float *s_shift = s_scale + MAX_OC_SMEM;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  const int pair_m_tiles = (p.m_tiles + 1) >> 1;
  const int total_tiles = pair_m_tiles * p.n_tiles;            // tiles of 256 pixels x BN channels
  const int first = blockIdx.x >> 1, step = gridDim.x >> 1;    // this cluster's tile walk

  if (threadIdx.x == 0) {
    ELB_TRACE(0);
    for (int i = 0; i < p.stride * p.stride; ++i) tma_prefetch_desc(&p.tmap[i]);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&pfull[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 2 * NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  for (int i = threadIdx.x; i < p.OCB * V; i += NUM_THREADS) {
    s_scale[i] = p.scale[i];
    s_shift[i] = p.shift[i];
  }
  if (warp == 1) tmem_alloc2(tmem_slot, TMEM_COLS);       // both CTAs take part in a cta_group::2 allocation
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                     // the peer's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int fail_code = 0;
  if (threadIdx.x == 0) ELB_TRACE(1);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    uint32_t it = 0;
    bool ok = true;
    for (int tile = first; tile < total_tiles && ok; tile += step) {
      const int pmt = tile / p.n_tiles, nt = tile % p.n_tiles;
      const int mt = 2 * pmt + static_cast<int>(rank);
      const bool live = mt < p.m_tiles;                     // an odd tile count leaves the last peer without pixels
      const int per_img = p.tiles_h * p.tiles_w;
      const int n0 = live ? mt / per_img : 0;
      const int r = live ? mt - n0 * per_img : 0;
      const int oh0 = (r / p.tiles_w) * p.BH, ow0 = (r % p.tiles_w) * p.BW;
      const int ks0 = p.rotate_k ? tile % p.k_stages : 0;
      for (int ki = 0; ki < p.k_stages; ++ki, ++it) {
        const int ks = ki + ks0 < p.k_stages ? ki + ks0 : ki + ks0 - p.k_stages;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait_warp(&empty[s], ph ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_PRODUCER; break; }
        uint8_t *a_dst = smem + s * L::STAGE_BYTES;
        uint8_t *b_dst = a_dst + L::A_BYTES;
        // weight image: [n tile][k stage][half][KC][BN/2 rows][16]
        const int8_t *b_src = p.wpack + ((static_cast<size_t>(nt) * p.k_stages + ks) * 2 + rank) * L::B_BYTES;
        const int q0 = ks * KC;
        const int valid = min(KC, p.Q - q0);
        if (lane == 0)
          mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>((live ? valid * (BM * 16) : 0) + L::B_BYTES));
        __syncwarp();
        if (lane == KC) tma_bulk_g2s(b_dst, b_src, L::B_BYTES, &full[s]);
        const int q = q0 + lane * p.box_c;
        if (live && lane * p.box_c < valid) {
          const int tap = q / p.CB, cb0 = q - tap * p.CB;
          const int kh = tap / p.KW, kw = tap - kh * p.KW;
          const int eh = kh - p.pad_t, ew = kw - p.pad_l;
          const int dh = (eh >= 0) ? eh / p.stride : -((-eh + p.stride - 1) / p.stride);
          const int dw = (ew >= 0) ? ew / p.stride : -((-ew + p.stride - 1) / p.stride);
          const int par_h = eh - dh * p.stride, par_w = ew - dw * p.stride;
          const CUtensorMap *tm = &p.tmap[par_h * p.stride + par_w];
          uint8_t *dst = a_dst + lane * p.box_c * (BM * 16);
          if (p.merged_rows) tma_tile_4d(dst, tm, (ow0 + dw) * 2, oh0 + dh, cb0, n0, &full[s]);
          else tma_tile_5d(dst, tm, 0, ow0 + dw, oh0 + dh, cb0, n0, &full[s]);
        }
        __syncwarp();
        if (lane == 0 && it < 16) ELB_TRACE(2 + it);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------------------------------------------------------- MMA issuer (leader CTA)
      constexpr uint32_t IDESC = umma_idesc(/*c s32*/ 2, /*a u8*/ 0, /*b s8*/ 1, 2 * BM, BN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = first; tile < total_tiles && ok; tile += step, ++tcount) {
        const uint32_t b = tcount & 1u, tph = (tcount >> 1) & 1u;
        if (!mbar_wait(&tempty[b], tph ^ 1u, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + b * BN;
        const int ks0 = p.rotate_k ? tile % p.k_stages : 0;
        for (int ki = 0; ki < p.k_stages; ++ki, ++it) {
          const int ks = ki + ks0 < p.k_stages ? ki + ks0 : ki + ks0 - p.k_stages;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, abort_flag) || !mbar_wait(&pfull[s], ph, abort_flag)) {
            ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break;
          }
          tc_fence_after_sync();
          if (it < 16) ELB_TRACE(20 + it);
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
          const int pairs = (min(KC, p.Q - ks * KC) + 1) >> 1;
#pragma unroll
          for (int k2 = 0; k2 < KC / 2; ++k2) {
            if (k2 < pairs) {
              // the same shared-memory offsets are read in both CTAs: 128 pixel rows and BN/2 weight rows each
              const uint64_t ad = umma_desc_kmajor(a_addr + k2 * 2 * (BM * 16), BM * 16, 128);
              const uint64_t bd = umma_desc_kmajor(b_addr + k2 * 2 * ((BN / 2) * 16), (BN / 2) * 16, 128);
              umma_i8_2cta(d_tmem, ad, bd, IDESC, (ki | k2) != 0 ? 1u : 0u);
            }
          }
          umma_commit_2cta(&empty[s]);       // frees the stage in both CTAs
        }
        if (ok) umma_commit_2cta(&tfull[b]);  // accumulators complete in both CTAs
        if (tcount == 0) ELB_TRACE(40);
      }
    } else if (lane == 0) {
      // ---------------------------------------------------------------- forwarder (peer CTA)
      uint32_t it = 0;
      bool ok = true;
      for (int tile = first; tile < total_tiles && ok; tile += step) {
        for (int ki = 0; ki < p.k_stages; ++ki, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_MMA; break; }
          mbar_arrive_cluster(mapa_u32(&pfull[s], 0));
          if (it < 16) ELB_TRACE(20 + it);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int elt = p.rq.out_type == OUT_F32 ? 4 : 1;
    const uint32_t tempty_leader0 = mapa_u32(&tempty[0], 0), tempty_leader1 = mapa_u32(&tempty[1], 0);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = first; tile < total_tiles && ok; tile += step, ++tcount) {
      const int pmt = tile / p.n_tiles, nt = tile % p.n_tiles;
      const int mt = 2 * pmt + static_cast<int>(rank);
      const uint32_t b = tcount & 1u, tph = (tcount >> 1) & 1u;
      const int per_img = p.tiles_h * p.tiles_w;
      const int n = mt / per_img;
      const int r = mt - n * per_img;
      const int oh = (r / p.tiles_w) * p.BH + row / p.BW;
      const int ow = (r % p.tiles_w) * p.BW + row % p.BW;
      const bool valid = mt < p.m_tiles && oh < p.OH && ow < p.OW;
      const size_t pix_off = (static_cast<size_t>(n) * p.OCB * p.OH + oh) * p.OW + ow;
      const size_t blk_stride = static_cast<size_t>(p.OH) * p.OW;
      if (!mbar_wait_warp(&tfull[b], tph, abort_flag)) { ok = false; fail_code = ST_WAIT_TIMEOUT_EPILOGUE; break; }
      tc_fence_after_sync();
      if (tcount == 0 && threadIdx.x == 64) ELB_TRACE(41);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * BN;
      auto emit = [&](int ob, const uint32_t (&rr)[16]) {
        const int ocb = nt * (BN / 16) + ob;
        if (valid && ocb < p.OCB) {
          int acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = static_cast<int>(rr[i]);
          const size_t off = (pix_off + ocb * blk_stride) * 16;
          if (p.acc_dump) {
            int4 *d = reinterpret_cast<int4 *>(p.acc_dump + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) d[i] = make_int4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
          }
          requant_store16(acc, s_scale + ocb * 16, s_shift + ocb * 16, static_cast<uint8_t *>(p.out) + off * elt, p.rq);
        }
      };
      constexpr int P = NUM_EPI_WARPS / 4;
      const int nblk = (BN / 16 - half + P - 1) / P;
      const uint32_t w_addr = t_addr + half * 16;
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
      // one arrival per warp on the LEADER's barrier: the accumulator is reused by MMAs that write
      // both CTAs' tensor memory
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(b ? tempty_leader1 : tempty_leader0);
      if (tcount == 0 && threadIdx.x == 64) ELB_TRACE(42);
    }
  }

  // ------------------------------------------------------------------ teardown
  if (fail_code != 0) atomicCAS(p.status, 0, fail_code);
  if (threadIdx.x == 0) ELB_TRACE(43);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // nobody leaves (or frees tensor memory) while the other CTA may still signal it
  tc_fence_after_sync();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) ELB_TRACE(44);
}

template <int BN, int KC, int STAGES>
cudaError_t launch_cfg2(const I8ConvParams &p, int num_sms, cudaStream_t s, bool attr_only, int *max_clusters) {
  using L = Smem2<BN, KC, STAGES>;
  auto kern = i8_umma2_kernel<BN, KC, STAGES>;
  if (attr_only) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return e;
    // how many 2-CTA clusters of this kernel the device can hold at once
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (num_sms / 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); n = num_sms / 2; }
    if (max_clusters) *max_clusters = n > 0 ? n : 1;
    return cudaSuccess;
  }
  const int tiles = ((p.m_tiles + 1) / 2) * p.n_tiles;
  int clusters = tiles < *max_clusters ? tiles : *max_clusters;
  kern<<<2 * clusters, NUM_THREADS, L::TOTAL, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

size_t i8_umma2_stage_b_bytes(int BN, int KC) { return static_cast<size_t>(KC) * (BN / 2) * 16; }

static cudaError_t dispatch2(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s, bool attr_only,
                             int *max_clusters) {
  if (cfg.BN == 256) return launch_cfg2<256, 8, 6>(p, num_sms, s, attr_only, max_clusters);
  if (cfg.BN == 128) return launch_cfg2<128, 8, 8>(p, num_sms, s, attr_only, max_clusters);
  return launch_cfg2<64, 8, 8>(p, num_sms, s, attr_only, max_clusters);
}

cudaError_t init_i8_umma2(I8UmmaConfig &cfg, int num_sms) {
  I8ConvParams dummy{};
  return dispatch2(dummy, cfg, num_sms, nullptr, true, &cfg.max_clusters);
}

cudaError_t launch_i8_umma2(const I8ConvParams &p, const I8UmmaConfig &cfg, int num_sms, cudaStream_t s) {
  if (p.OCB * V > MAX_OC_SMEM) return cudaErrorInvalidValue;
  int mc = cfg.max_clusters;
  return dispatch2(p, cfg, num_sms, s, false, &mc);
}

}  // namespace elb
