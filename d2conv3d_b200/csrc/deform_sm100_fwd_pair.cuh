// Forward kernel for CTA pairs (cluster of 2, tcgen05 cta_group::2).  Included by deform_sm100_fwd.cu after
// the single-CTA kernel, whose constants, FwdParams and gather helpers it shares.
//
// Why pairs: with one CTA per 128-voxel tile every work unit streams a whole Cout x 64 weight slice (64 KB for
// Cout = 512) from L2 for only 128 rows of A, and that stream alone takes 0.43 ms of the 0.70 ms kernel for the
// headline shape.  A pair computes M = 256 (two tiles, each CTA gathers its own 128 rows) against ONE weight
// slice split between the two CTAs: each CTA loads, and holds in shared memory, only Cout/2 rows per unit, so
// the weight traffic per SM halves and the ring gets twice the depth in the same space.
//
// Unit of work: (tile pair tp, slice s); clusters own contiguous unit ranges (stream-K).  CTA `rank` of the pair
// works on tile 2*tp + rank (a missing odd tile is an all-zero A tile whose rows are never stored).
//
// Signalling (all waits bounded):
//   a_full[s]   leader's barrier, 2 x 16 arrivals: local gather warps + the peer's (remote arrive)
//   b_full[s]   own barrier per CTA (bulk-copy bytes); the peer's idle MMA warp forwards its completion to the
//               leader's b_full[s], which therefore counts 2 arrivals + the leader's bytes
//   a_empty[s], b_empty[s], acc_full   one barrier per CTA; the leader commits to its own and to the peer's
//   acc_empty   leader's barrier, 2 x 4 arrivals (both epilogues)
#pragma once

namespace pair {

constexpr int kBlockRows = 128;    // weight rows per CTA per 256-wide N block

struct PairParams {
  FwdParams f;
  int n_tile_pairs;
  long long n_pair_units;
  int b_stages, b_half_bytes;      // ring depth, bytes per CTA per unit (= Cout/2 rows x 128 B)
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fwd_sm100_pair_kernel(const PairParams pp) {
  const FwdParams& p = pp.f;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const int rec_off = kAStages * kAStageBytes + pp.b_stages * pp.b_half_bytes;
  const int bar_off = rec_off + kRStages * kRStageBytes;
  const uint32_t a_base = base, b_base = base + kAStages * kAStageBytes, rec_base = base + rec_off,
                 bar_base = base + bar_off;
  // barrier slots: a_full 0-3, a_empty 4-7, b_full 8-11, b_empty 12-15, acc_full 16, acc_empty 17,
  // (18: tmem slot + abort flag), r_full 19-22, r_empty 23-26
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (4 + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (8 + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (12 + s); };
  const uint32_t acc_full = bar_base + 8u * 16, acc_empty = bar_base + 8u * 17;
  auto r_full = [&](int s) { return bar_base + 8u * (19 + s); };
  auto r_empty = [&](int s) { return bar_base + 8u * (23 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * 18 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  const Geom& g = p.g;
  const long long cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
  const long long u_beg = pp.n_pair_units * cid / ncl, u_end = pp.n_pair_units * (cid + 1) / ncl;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(a_full(s), 2 * kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < pp.b_stages; ++s) { ptx::mbar_init(b_full(s), leader ? 2 : 1); ptx::mbar_init(b_empty(s), 1); }
    for (int s = 0; s < kRStages; ++s) { ptx::mbar_init(r_full(s), 1); ptx::mbar_init(r_empty(s), kGatherWarps); }
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_empty, 2 * kEpiWarps);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc_pair(ptx::smem_u32((const void*)tmem_slot), (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();       // both CTAs' barriers exist before anyone arrives remotely
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // coordinates of pair unit u for THIS CTA
  auto unit_tile = [&](long long u, int& s, int& b, int& v0, bool& tile_ok) {
    const int tp = (int)(u / p.S);
    s = (int)(u % p.S);
    const int tile = 2 * tp + (int)rank;
    tile_ok = tile < p.n_tiles;
    b = tile_ok ? tile / p.tiles_per_clip : 0;
    v0 = tile_ok ? (tile % p.tiles_per_clip) * kBM : 0;
  };

  if (warp < kEpiWarps) {
    // ===================== epilogue: one pass per tile-pair segment =====================
    const uint32_t acc_empty_leader = ptx::mapa_shared(acc_empty, 0);
    int seg = 0;
    for (long long u = u_beg; u < u_end; ++seg) {
      const int s_beg = (int)(u % p.S);
      const int s_end = (int)min((long long)p.S, s_beg + (u_end - u));
      int s_, b, v0; bool tile_ok;
      unit_tile(u, s_, b, v0, tile_ok);
      u += s_end - s_beg;
      const bool whole = (s_beg == 0 && s_end == p.S);
      if (!ptx::mbar_wait_cluster(acc_full, seg & 1, abort_flag, 2000)) break;
      ptx::tc_fence_after();
      const int v = v0 + warp * 32 + lane;
      float* yb = p.y + (long long)b * g.Cout * g.V + v;
      for (int c0 = 0; c0 < p.N; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
        if (tile_ok && v < g.V) {
          if (whole) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bb = p.bias ? __ldg(p.bias + c0 + j) : 0.f;
              yb[(long long)(c0 + j) * g.V] = __uint_as_float(r[j]) + bb;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bb = (p.bias && s_beg == 0) ? __ldg(p.bias + c0 + j) : 0.f;
              atomicAdd(yb + (long long)(c0 + j) * g.V, __uint_as_float(r[j]) + bb);
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(acc_empty_leader);
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && leader) {
      // ===================== MMA issuer (leader CTA only) =====================
      const uint32_t acc_full_peer = ptx::mapa_shared(acc_full, 1);
      int seg = 0;
      uint32_t k = 0;
      bool ok = true;
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int s_beg = (int)(u % p.S);
        const int s_end = (int)min((long long)p.S, s_beg + (u_end - u));
        u += s_end - s_beg;
        if (!ptx::mbar_wait_cluster(acc_empty, (seg & 1) ^ 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int s = s_beg; s < s_end; ++s, ++k) {
          const int sa = k % kAStages, sb = k % pp.b_stages;
          if (!ptx::mbar_wait_cluster(a_full(sa), (k / kAStages) & 1, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait_cluster(b_full(sb), (k / pp.b_stages) & 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t adesc = ptx::umma_desc_kmajor_sw128(a_base + sa * kAStageBytes);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            for (int n0 = 0, nb = 0; n0 < p.N; n0 += 256, ++nb) {
              const int nc = min(256, p.N - n0);
              const uint64_t bdesc =
                  ptx::umma_desc_kmajor_sw128(b_base + sb * pp.b_half_bytes + nb * (kBlockRows * 128));
              ptx::umma_bf16_pair(tmem_base + (uint32_t)n0, adesc + (uint64_t)(2 * kk), bdesc + (uint64_t)(2 * kk),
                                  ptx::umma_idesc_bf16_f32(2 * kBM, nc), (s > s_beg || kk > 0) ? 1u : 0u);
            }
          }
          ptx::umma_commit_pair(a_empty(sa));
          ptx::umma_commit_pair(ptx::mapa_shared(a_empty(sa), 1));
          ptx::umma_commit_pair(b_empty(sb));
          ptx::umma_commit_pair(ptx::mapa_shared(b_empty(sb), 1));
        }
        if (ok) {
          ptx::umma_commit_pair(acc_full);
          ptx::umma_commit_pair(acc_full_peer);
        }
      }
    } else if (lane == 0) {
      // ===================== peer: forward "my weight half has landed" to the leader =====================
      uint32_t k = 0;
      for (long long u = u_beg; u < u_end; ++u, ++k) {
        const int sb = k % pp.b_stages;
        if (!ptx::mbar_wait(b_full(sb), (k / pp.b_stages) & 1, abort_flag, 100)) break;
        ptx::mbar_arrive_cluster(ptx::mapa_shared(b_full(sb), 0));
      }
    }
  } else if (warp == kLoadWarp) {
    // ===================== weight loader: this CTA's rows of every 256-wide N block =====================
    if (lane == 0) {
      uint32_t k = 0;
      for (long long u = u_beg; u < u_end; ++u, ++k) {
        const int s = (int)(u % p.S), sb = k % pp.b_stages;
        if (!ptx::mbar_wait_cluster(b_empty(sb), ((k / pp.b_stages) & 1) ^ 1, abort_flag, 200)) break;
        ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)pp.b_half_bytes);
        const uint8_t* src = p.w_sw + (long long)s * p.b_stage_bytes;
        const uint32_t dst = b_base + sb * pp.b_half_bytes;
        for (int n0 = 0, nb = 0; n0 < p.N; n0 += 256, ++nb) {
          const int rows = min(256, p.N - n0) / 2;
          ptx::bulk_g2s(dst + nb * (kBlockRows * 128), src + (long long)(n0 + (int)rank * rows) * 128,
                        (uint32_t)rows * 128u, b_full(sb));
        }
      }
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)pp.b_stages ? issued - pp.b_stages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(q % pp.b_stages), (q / pp.b_stages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
  } else if (warp == kRecWarp) {
    // ===================== gather-record loader (own tile) =====================
    if (lane == 0) {
      uint32_t k = 0;
      for (long long u = u_beg; u < u_end; ++u, ++k) {
        int s, b, v0; bool tile_ok;
        unit_tile(u, s, b, v0, tile_ok);
        const int gt = s / p.nh, tap = gt % g.K, grp = gt / g.K;
        const int sr = k % kRStages;
        if (!ptx::mbar_wait(r_empty(sr), ((k / kRStages) & 1) ^ 1, abort_flag, 200)) break;
        const int rows = tile_ok ? min(kBM, g.V - v0) : 0;
        uint8_t* hdr = base_ptr + rec_off + sr * kRStageBytes + kRecBytes;
        *reinterpret_cast<long long*>(hdr) = (long long)b * g.Vin * g.Cin + grp * g.cpg + (s % p.nh) * kBK;
        *reinterpret_cast<int*>(hdr + 8) = rows;
        if (tile_ok) {
          const uint32_t bytes = (uint32_t)rows * 48u;
          ptx::mbar_arrive_expect_tx(r_full(sr), bytes);
          ptx::bulk_g2s(rec_base + sr * kRStageBytes,
                        p.recs + 3 * ((((long long)b * g.G + grp) * g.K + tap) * g.V + v0), bytes, r_full(sr));
        } else {
          ptx::mbar_arrive(r_full(sr));
        }
      }
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)kRStages ? issued - kRStages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(r_full(q % kRStages), (q / kRStages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
  } else {
    // ===================== gather producers (own tile; arrive on the leader's a_full) =====================
    const int t = threadIdx.x - kGatherWarp0 * 32;
    const int j = t & 7;
    const int r0 = t >> 3;
    uint32_t row_dst[kRowsPerThread];
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const int r = r0 + kRowStride * i;
      row_dst[i] = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
    }
    const uint32_t a_full_leader[kAStages] = {ptx::mapa_shared(a_full(0), 0), ptx::mapa_shared(a_full(1), 0),
                                              ptx::mapa_shared(a_full(2), 0), ptx::mapa_shared(a_full(3), 0)};
    const uint32_t n_my_units = (uint32_t)(u_end - u_beg);
    for (uint32_t k = 0; k < n_my_units; ++k) {
      const int sr = k % kRStages, sa = k % kAStages;
      if (!ptx::mbar_wait(r_full(sr), (k / kRStages) & 1, abort_flag)) break;
      const uint8_t* rec_stage = base_ptr + rec_off + sr * kRStageBytes;
      const __half* xb = reinterpret_cast<const __half*>(p.x_cl) + *reinterpret_cast<const long long*>(rec_stage + kRecBytes) + j * 8;
      const int rows = *reinterpret_cast<const int*>(rec_stage + kRecBytes + 8);
      uint4 c[kRowsPerThread][8];
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i) {
        const int r = r0 + kRowStride * i;
        uint2 head = make_uint2(0u, 0u);
        if (r < rows) head = *reinterpret_cast<const uint2*>(rec_stage + r * 48);
        load_corners(xb, p.cs, head.x, head.y, c[i]);
      }
      if (!ptx::mbar_wait_cluster(a_empty(sa), ((k / kAStages) & 1) ^ 1, abort_flag)) break;
      const uint32_t stage = a_base + sa * kAStageBytes;
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i) {
        const int r = r0 + kRowStride * i;
        uint4 w03 = make_uint4(0u, 0u, 0u, 0u), w47 = w03;
        if (r < rows) {
          w03 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
          w47 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 32);
        }
        blend_store(c[i], w03, w47, stage + row_dst[i]);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive_cluster(a_full_leader[sa]);
        ptx::mbar_arrive(r_empty(sr));
      }
    }
  }

  // ---- teardown: neither CTA may free tensor memory or exit while the other can still touch it ----
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace pair
