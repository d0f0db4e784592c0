// The single-CTA forward kernel (included by deform_sm100_fwd.cu, whose constants, FwdParams and gather helpers it
// uses).  Warp roles are aligned to warpgroups (4 epilogue warps | MMA, weight loader, record loader, one idle warp
// | 16 gather warps) so that `setmaxnreg` can move registers from the light roles to the gather warps, whose loop
// is software-pipelined at row granularity (see the producer branch).
// Optional instrumentation (compiled in with -DD2C_UNIT_TRACE, `python -m d2conv3d_b200.build --unit-trace`): every
// role of ONE CTA stamps clock64() at fixed points of its per-unit loop for a window of 64 units, and every CTA
// records its start / end (globaltimer), its SM and its unit count.  Read with `python -m d2conv3d_b200.unit_trace`.
// Layout of the buffer (long long): [role 0..4][unit 0..63][event 0..7], then [CTA][t0, t1, smid, units].
// Roles: 0 record loader, 1 weight loader, 2 MMA issuer, 3 / 4 first / last gather warp (lane 0).
#ifdef D2C_UNIT_TRACE
#define D2C_TR(role, k, e)                                                                                    \
  do {                                                                                                        \
    if (p.trace && (int)blockIdx.x == p.trace_cta && (int)(k) >= p.trace_k0 && (int)(k) < p.trace_k0 + 64)    \
      p.trace[((role) * 64 + ((int)(k) - p.trace_k0)) * 8 + (e)] = clock64();                                 \
  } while (0)
#else
#define D2C_TR(role, k, e) ((void)0)
#endif

constexpr int kThreadsFwd = 24 * 32;
static_assert(128 * 56 + 128 * 40 + 512 * 96 <= kThreadsFwd * 80, "setmaxnreg budget exceeds the CTA's register allocation");
constexpr int kMmaWarpFwd = 4, kLoadWarpFwd = 5, kRecWarpFwd = 6, kGatherWarp0Fwd = 8;

// kX3 = 0: math mode bf16 (a unit is 64 channels of one tap, one bf16 operand pair).
// kX3 = 1: math mode bf16x3, the fp32-parity mode: a unit is 32 channels; the A row holds [hi(32) | lo(32)] of
//          the fp32 blend, the weight row [hi(32) | lo(32)] of the fp32 weight, and the issuer forms
//          a_hi*b_hi + a_lo*b_hi + a_hi*b_lo from the 16-channel K sub-blocks of the same two tiles.
// kDual = 1 (single-pass mode only): 32 channels per offset group, a 64-channel unit spans two groups.
// kSave = 1: the blended tiles are also written to FwdParams::sav (a forward whose backward will follow).  A template
//          parameter, not a run-time test, so that the inference kernel carries neither the stores nor the registers
//          for their addresses.
template <int kX3, int kDual, int kSave>
__global__ void __launch_bounds__(kThreadsFwd, 1)
fwd_sm100_kernel(const FwdParams p) {
  constexpr int kUnitCh = kX3 ? 32 : 64;
  constexpr int kRStage = (1 + kDual) * kRecBytes + 16;      // record set(s) + unit header
  constexpr int hdr_off = (1 + kDual) * kRecBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const int rec_off = kAStages * kAStageBytes + p.b_stages * p.b_stage_bytes;
  const int bar_off = rec_off + kRStages * kRStage;
  const uint32_t a_base = base, b_base = base + kAStages * kAStageBytes, rec_base = base + rec_off,
                 bar_base = base + bar_off;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (kAStages + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * kAStages + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * kAStages + 4 + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * kAStages + 8);
  const uint32_t acc_empty = bar_base + 8u * (2 * kAStages + 9);
  auto r_full = [&](int s) { return bar_base + 8u * (2 * kAStages + 11 + s); };
  auto r_empty = [&](int s) { return bar_base + 8u * (2 * kAStages + 11 + kRStages + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * (2 * kAStages + 10));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * (2 * kAStages + 10) + 4);

#ifdef D2C_UNIT_TRACE
  unsigned long long cta_t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(cta_t0));
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Geom& g = p.g;
  // A CTA's work is n_parts (<= 16) contiguous unit ranges, one inside every clip (cta_part_range in
  // deform_sm100_fwd.cu); ring slots, phases and segment counters run on across the parts, positions restart at every
  // part.  Thread 0 puts the ranges into shared memory once, so that the roles (some of them left with 40 registers)
  // do no 64-bit division.
  // (unit indices fit 31 bits: checked by the host)
  int* part_tab = reinterpret_cast<int*>(base_ptr + bar_off + 256);      // [part][beg, end], then the total
  // Large volumes (FwdParams::rr): whole tiles dealt round-robin instead -- at any time the CTAs then work on
  // gridDim.x CONSECUTIVE tiles, whose sampling neighbourhoods overlap, so the part of the staged input they gather
  // from is a few planes and not a few planes around 148 places spread over the whole volume (which L2 cannot hold:
  // the stride-4 decoder layer re-fetched its 210 MB input 22 times).
  auto part_range = [&](int part, int& beg, int& end) {
    if (p.rr) {
      const int tile = part * (int)gridDim.x + (int)blockIdx.x;
      beg = tile * p.S;
      end = tile < p.n_tiles ? beg + p.S : beg;
    } else {
      beg = part_tab[2 * part];
      end = part_tab[2 * part + 1];
    }
  };

  if (threadIdx.x == 0) {
    int total = 0;
    if (p.rr) {
      // round-robin tiles: part r is tile r * gridDim.x + blockIdx.x (computed where it is needed)
      for (int tile = (int)blockIdx.x; tile < p.n_tiles; tile += (int)gridDim.x) total += p.S;
    } else {
      for (int part = 0; part < p.n_parts; ++part) {
        long long pb, pe;
        cta_part_range(p, part, pb, pe);
        part_tab[2 * part] = (int)pb; part_tab[2 * part + 1] = (int)pe;
        total += (int)(pe - pb);
      }
    }
    part_tab[32] = total;
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(a_full(s), kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < p.b_stages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    for (int s = 0; s < kRStages; ++s) { ptx::mbar_init(r_full(s), 1); ptx::mbar_init(r_empty(s), kGatherWarps); }
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_empty, kEpiWarps);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc(ptx::smem_u32((const void*)tmem_slot), (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Register re-balancing between the roles (warpgroup-wide, first statement of each role's branch): the epilogue
  // and service warps give registers back, the gather warps take them, so that a gather thread can hold the corner
  // loads of TWO rows in flight while it blends.  The increase is served from what the CTA itself gave back: the CTA
  // is launched with 768 x 80 = 61440 registers and 128*56 + 128*40 + 512*96 = 61440 (asking for more would make
  // the increase wait for registers that never come).
  if (warp < kEpiWarps) {
    // ===================== epilogue: one pass per tile segment =====================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    int seg = 0;
    for (int part = 0; part < p.n_parts; ++part) {
    if (*abort_flag) break;
    int u_beg, u_end;
    part_range(part, u_beg, u_end);
    for (int u = u_beg; u < u_end; ++seg) {
      const int tile = u / p.S, s_beg = u % p.S;
      const int s_end = min(min(p.S, s_beg + (u_end - u)), s_beg + p.seg_cap);
      u += s_end - s_beg;
      const bool whole = (s_beg == 0 && s_end == p.S);
      const int b = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
      if (!ptx::mbar_wait(acc_full, seg & 1, abort_flag, 2000)) break;
      ptx::tc_fence_after();
      const int v = v0 + warp * 32 + lane;
      float* yb = p.y + (long long)b * g.Cout * g.V + v;
      if ((g.V & 3) == 0) {
        // Each lane holds 32 channels of ONE voxel; y is [clip][channel][voxel], so a lane's values lie V floats
        // apart.  A 4 x 4 transpose inside every lane quad (two shuffle stages) gives lane q of the quad channel
        // 4i + q of the quad's four consecutive voxels: 16-byte stores / vector reductions, a quarter of the memory
        // instructions (the partial-tile epilogue was bound by their issue, not by bytes).
        const int q = lane & 3;
        const int vq = v0 + warp * 32 + (lane & ~3);
        float* yq = p.y + (long long)b * g.Cout * g.V + vq;
        const bool live = vq < g.V;                      // V is a multiple of 4: a quad is valid or invalid as a whole
        for (int c0 = 0; c0 < p.N; c0 += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t* a = r + 4 * i;
            const uint32_t t0 = __shfl_xor_sync(0xffffffffu, (q & 1) ? a[0] : a[1], 1);
            const uint32_t t1 = __shfl_xor_sync(0xffffffffu, (q & 1) ? a[2] : a[3], 1);
            if (q & 1) { a[0] = t0; a[2] = t1; } else { a[1] = t0; a[3] = t1; }
            const uint32_t u0 = __shfl_xor_sync(0xffffffffu, (q & 2) ? a[0] : a[2], 2);
            const uint32_t u1 = __shfl_xor_sync(0xffffffffu, (q & 2) ? a[1] : a[3], 2);
            if (q & 2) { a[0] = u0; a[1] = u1; } else { a[2] = u0; a[3] = u1; }
            if (live) {
              const int c = c0 + 4 * i + q;
              const float bb = (p.bias && (whole || s_beg == 0)) ? __ldg(p.bias + c) : 0.f;
              float* dst = yq + (long long)c * g.V;
              const float f0 = __uint_as_float(a[0]) + bb, f1 = __uint_as_float(a[1]) + bb,
                          f2 = __uint_as_float(a[2]) + bb, f3 = __uint_as_float(a[3]) + bb;
              if (whole)
                *reinterpret_cast<float4*>(dst) = make_float4(f0, f1, f2, f3);
              else
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(f0), "f"(f1), "f"(f2), "f"(f3)
                             : "memory");
            }
          }
        }
      } else {
      for (int c0 = 0; c0 < p.N; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
        if (v < g.V) {
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
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty);
    }
    }
  } else if (warp < kGatherWarp0Fwd) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
   if (warp == kMmaWarpFwd) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      // One thread drives the tensor core, so its own instruction latency is on the critical path of every unit:
      // no integer division or modulo by run-time values in the per-unit path (ring slots and phases are carried as
      // counters), descriptors are built from constants hoisted out of the loops.
      int seg = 0;
      uint32_t k = 0;           // units consumed so far (A and B rings advance together)
      int sb = 0;               // weight-ring slot of unit k and its phase
      uint32_t phb = 0;
      bool ok = true;
      constexpr int kSteps = kX3 ? 6 : 4;
      // K sub-blocks (16 channels = 32 bytes) of the A and B rows that meet in each MMA
      constexpr int ka_[6] = {0, 1, kX3 ? 2 : 2, kX3 ? 3 : 3, 0, 1};   // bf16: (k,k); x3: hi*hi, lo*hi, hi*lo
      constexpr int kb_[6] = {0, 1, kX3 ? 0 : 2, kX3 ? 1 : 3, 2, 3};
      const int n_halves = (p.N + 255) / 256;
      const uint32_t idesc_full = ptx::umma_idesc_bf16_f32(kBM, 256);
      const uint32_t idesc_last = ptx::umma_idesc_bf16_f32(kBM, p.N - (n_halves - 1) * 256);
      const uint64_t adesc0 = ptx::umma_desc_kmajor_sw128(a_base), bdesc0 = ptx::umma_desc_kmajor_sw128(b_base);
      const uint64_t a_step = (uint64_t)(kAStageBytes >> 4), b_step = (uint64_t)(p.b_stage_bytes >> 4);
      for (int part = 0; ok && part < p.n_parts; ++part) {
      if (*abort_flag) break;
      int u_beg, u_end;
    part_range(part, u_beg, u_end);
      int s_beg = u_beg % p.S;                                          // once per part
      for (int u = u_beg; ok && u < u_end; ++seg) {
        const int s_end = min(min(p.S, s_beg + (u_end - u)), s_beg + p.seg_cap);
        u += s_end - s_beg;
        if (!ptx::mbar_wait(acc_empty, (seg & 1) ^ 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int s = s_beg; s < s_end; ++s, ++k) {
          const int sa = k & (kAStages - 1);
          D2C_TR(2, k, 0);
          if (!ptx::mbar_wait(a_full(sa), (k / kAStages) & 1, abort_flag)) { ok = false; break; }
          D2C_TR(2, k, 1);
          if (!ptx::mbar_wait(b_full(sb), phb, abort_flag)) { ok = false; break; }
          D2C_TR(2, k, 2);
          ptx::tc_fence_after();
          // descriptor address fields count 16-byte units: a stage further along adds stage_bytes / 16
          const uint64_t adesc = adesc0 + a_step * (uint64_t)sa;
          const uint64_t bdesc = bdesc0 + b_step * (uint64_t)sb;
#pragma unroll
          for (int kk = 0; kk < kSteps; ++kk) {
            for (int h = 0; h < n_halves; ++h)
              ptx::umma_bf16(tmem_base + (uint32_t)(h * 256), adesc + (uint64_t)(2 * ka_[kk]),
                             bdesc + (uint64_t)(h * (256 * 128 / 16)) + (uint64_t)(2 * kb_[kk]),
                             h + 1 < n_halves ? idesc_full : idesc_last, (s > s_beg || kk > 0) ? 1u : 0u);
          }
          D2C_TR(2, k, 3);
          ptx::umma_commit(a_empty(sa));
          ptx::umma_commit(b_empty(sb));
          D2C_TR(2, k, 4);
          if (++sb == p.b_stages) { sb = 0; phb ^= 1u; }
        }
        if (ok) ptx::umma_commit(acc_full);
        s_beg = s_end == p.S ? 0 : s_end;
      }
      }
    }
  } else if (warp == kLoadWarpFwd) {
    // ===================== weight-slice loader =====================
    if (lane == 0) {
      uint32_t k = 0;
      int sb = 0;                       // ring slot and phase as counters: no division in the per-unit path
      uint32_t phb = 1;                 // the wait for a FREE slot looks at the previous phase
      for (int part = 0; part < p.n_parts; ++part) {
      if (*abort_flag) break;
      int u_beg, u_end;
    part_range(part, u_beg, u_end);
      int s = u_beg % p.S;              // once per part
      const uint8_t* src = p.w_sw + (long long)s * p.b_stage_bytes;
      const int n_part_units = u_end - u_beg;
      for (int i = 0; i < n_part_units; ++i, ++k) {
        D2C_TR(1, k, 0);
        if (!ptx::mbar_wait(b_empty(sb), phb, abort_flag, 200)) break;
        D2C_TR(1, k, 1);
        ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)p.b_stage_bytes);
        const uint32_t dst = b_base + sb * p.b_stage_bytes;
        for (int off = 0; off < p.b_stage_bytes; off += 32768)
          ptx::bulk_g2s(dst + off, src + off, (uint32_t)min(32768, p.b_stage_bytes - off), b_full(sb));
        if (++sb == p.b_stages) { sb = 0; phb ^= 1u; }
        src += p.b_stage_bytes;
        if (++s == p.S) { s = 0; src = p.w_sw; }
      }
      }
      // never leave with a bulk copy in flight: wait (bounded) for the last copies issued
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)p.b_stages ? issued - p.b_stages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(q % p.b_stages), (q / p.b_stages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
  } else if (warp == kRecWarpFwd) {
    // ===================== gather-record loader =====================
    // The records of a unit's rows are one contiguous run of the [B][G][K][V] stream: one bulk copy per unit,
    // kRStages units ahead of the gather warps, so the producers read them from shared memory.
    if (lane == 0) {
      uint32_t k = 0;
      // position of the first unit, once per CTA; then everything advances by counters (this single thread's
      // instruction latency sits between "stage free" and "copy issued" for every unit: no division in the loop)
      const long long grp_ch = kDual ? 2 * g.cpg : g.cpg;
      const uint64_t pol_stream = ptx::l2_evict_first();       // records are read once
      for (int part = 0; part < p.n_parts; ++part) {
      if (*abort_flag) break;
      int u_beg, u_end;
    part_range(part, u_beg, u_end);
      int s = u_beg % p.S;
      const int tile0 = u_beg / p.S;
      int b = tile0 / p.tiles_per_clip, v0 = (tile0 % p.tiles_per_clip) * kBM;
      int tile = tile0;
      int h = s % p.nh, tap = (s / p.nh) % g.K, grp = (s / p.nh) / g.K;   // dual: grp is the index of a group PAIR
      const int n_part_units = u_end - u_beg;
      for (int i = 0; i < n_part_units; ++i, ++k) {
        const int sr = k & (kRStages - 1);
        D2C_TR(0, k, 0);
        if (!ptx::mbar_wait(r_empty(sr), ((k / kRStages) & 1) ^ 1, abort_flag, 200)) break;
        D2C_TR(0, k, 1);
        const int rows = min(kBM, g.V - v0);
        // unit header for the gather warps (no index arithmetic there); ordered before their reads by the
        // release of the arrive below and the acquire of their wait
        uint8_t* hdr = base_ptr + rec_off + sr * kRStage + hdr_off;
        *reinterpret_cast<long long*>(hdr) = (long long)b * g.Vin * g.Cin + grp * grp_ch + h * kUnitCh;
        *reinterpret_cast<int*>(hdr + 8) = rows;
        if constexpr (kSave) {
          // where this unit's samples go in the image kept for the weight gradient (8 KB blocks, see FwdParams)
          int word;
          if constexpr (kX3) {
            // 64-channel slice of the weight gradient that holds this 32-channel unit, and which half of it
            const int s64 = p.sav_pairg ? (grp >> 1) * g.K + tap : (grp * g.K + tap) * (p.nh >> 1) + (h >> 1);
            const int half = p.sav_pairg ? (grp & 1) : (h & 1);
            word = (((tile * 2 * p.sav_np + (s64 >> 1)) * 4 + (s64 & 1)) << 1) | half;
          } else {
            word = tile * 2 * (2 * p.sav_np) + s;
          }
          *reinterpret_cast<int*>(hdr + 12) = word;
        }
        const uint32_t bytes = (uint32_t)rows * 48u;
        ptx::mbar_arrive_expect_tx(r_full(sr), bytes * (uint32_t)(1 + kDual));
#pragma unroll
        for (int set = 0; set <= kDual; ++set) {
          const int og = kDual ? 2 * grp + set : grp;      // offset group whose records fill this set
          ptx::bulk_g2s_hint(rec_base + sr * kRStage + set * kRecBytes,
                             p.recs + 3 * ((((long long)b * g.G + og) * g.K + tap) * g.V + v0), bytes, r_full(sr), pol_stream);
        }
        // next unit: (h, tap, grp) count through the tile's slices, then the next tile of the clip / next clip
        if (++h == p.nh) {
          h = 0;
          if (++tap == g.K) { tap = 0; ++grp; }
        }
        if (++s == p.S) {
          s = 0; h = 0; tap = 0; grp = 0;
          ++tile;
          v0 += kBM;
          if (v0 >= p.tiles_per_clip * kBM) { v0 = 0; ++b; }
        }
      }
      }
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)kRStages ? issued - kRStages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(r_full(q % kRStages), (q / kRStages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
   }
  } else {
    // ===================== gather producers (software-pipelined) =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
    // A thread owns rows r0 and r0 + 64 of every unit, chunk j (16 B of the 128-byte A row).  Items are taken in
    // the order (unit k, row 0), (unit k, row 1), (unit k+1, row 0) ...; the 8 corner loads of item t+1 are
    // issued before item t is blended, so 8 loads are always in flight under the blend and 16 while it waits.
    const int t = threadIdx.x - kGatherWarp0Fwd * 32;
    const int j = t & 7;             // 16-byte chunk (8 channels) of the 128-byte row
    const int r0 = t >> 3;           // rows r0, r0 + kRowStride
    const uint32_t n_my_units = (uint32_t)part_tab[32];
    bool ok = true;
    // Samples kept for the weight gradient (p.sav != nullptr): the thread's two rows r0 and r0 + 64 are the same row
    // of the two 64-voxel blocks of the tile, so its byte offset inside an 8 KB block is fixed.
    const uint32_t sav_row = (uint32_t)((r0 >> 3) * 1024 + (r0 & 7) * 128);
    const uint64_t pol_stream = ptx::l2_evict_first();

    auto issue = [&](uint32_t k, int i, uint4 (&c)[8]) {
      const uint8_t* rec_base_ptr = base_ptr + rec_off + (k % kRStages) * kRStage;
      const long long xoff = *reinterpret_cast<const long long*>(rec_base_ptr + hdr_off);
      const int rows = *reinterpret_cast<const int*>(rec_base_ptr + hdr_off + 8);
      // dual: 16-byte chunks 4-7 of a row (channels 32-63 of the unit) belong to the second offset group
      const uint8_t* rec_stage = rec_base_ptr + ((kDual && j >= 4) ? kRecBytes : 0);
      const int r = r0 + kRowStride * i;
      uint2 head = make_uint2(0u, 0u);
      if (r < rows) head = *reinterpret_cast<const uint2*>(rec_stage + r * 48);
      if constexpr (kX3)
        load_corners_f32(reinterpret_cast<const float*>(p.x_cl) + xoff + j * 4, p.cs, head.x, head.y, c);
      else
        load_corners(reinterpret_cast<const __half*>(p.x_cl) + xoff + j * 8, p.cs, head.x, head.y, c);
    };
    // sd (kSave): where the 16 bytes this lane writes to the A tile (bf16x3: the lane pair's hi chunk or lo chunk) go
    // in the kept image
    auto consume = [&](uint32_t k, int i, const uint4 (&c)[8], uint8_t* sd) {
      const uint8_t* rec_base_ptr = base_ptr + rec_off + (k % kRStages) * kRStage;
      const int rows = *reinterpret_cast<const int*>(rec_base_ptr + hdr_off + 8);
      const uint8_t* rec_stage = rec_base_ptr + ((kDual && j >= 4) ? kRecBytes : 0);
      const uint32_t stage = a_base + (k % kAStages) * kAStageBytes;
      const int r = r0 + kRowStride * i;
      if constexpr (kX3) {
        float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // rows past the clip end: stage bytes are stale
        if (r < rows) {
          const uint2 w01 = *reinterpret_cast<const uint2*>(rec_stage + r * 48 + 8);
          const uint4 w25 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
          const uint2 w67 = *reinterpret_cast<const uint2*>(rec_stage + r * 48 + 32);
          w[0] = __uint_as_float(w01.x); w[1] = __uint_as_float(w01.y);
          w[2] = __uint_as_float(w25.x); w[3] = __uint_as_float(w25.y);
          w[4] = __uint_as_float(w25.z); w[5] = __uint_as_float(w25.w);
          w[6] = __uint_as_float(w67.x); w[7] = __uint_as_float(w67.y);
        }
        // item j = channels 4j..4j+3: hi in 16-byte chunk j/2 (half j&1), lo in chunk 4 + j/2; the lane pair (j, j^1)
        // shares both chunks: the even lane writes the hi chunk, the odd lane the lo chunk
        const uint32_t row_base = stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        const uint4 o = blend_split_store16(c, w, row_base + ((((j & 1) * 4 + (j >> 1)) ^ (r & 7)) << 4), (j & 1) != 0);
        if constexpr (kSave) ptx::stg_v4_hint(sd, o, pol_stream);
      } else {
        uint4 w03 = make_uint4(0u, 0u, 0u, 0u), w47 = w03;       // rows past the clip end: stage bytes are stale
        if (r < rows) {
          w03 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
          w47 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 32);
        }
        const uint4 o = blend_store(c, w03, w47, stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4)));
        if constexpr (kSave) ptx::stg_v4_hint(sd, o, pol_stream);
      }
    };

    uint4 c0[8], c1[8];
    if (n_my_units > 0) {
      ok = ptx::mbar_wait(r_full(0), 0, abort_flag);
      if (ok) issue(0, 0, c0);
    }
    for (uint32_t k = 0; ok && k < n_my_units; ++k) {
      const int sr = k % kRStages, sa = k % kAStages;
      // where this lane's bytes of the unit go in the kept image: block = (tile, 64-voxel block, slice) in the
      // single-pass mode; (tile, 64-voxel block, slice pair, {hi, lo}, slice of the pair) in the hi/lo mode, where a
      // 64-channel row holds this unit's 32 channels in its half `half`, an even lane holds the hi chunk of the lane
      // pair's 8 channels and an odd lane the lo chunk two blocks further.  The tile's second 64-voxel block (row 1 of
      // this thread) lies sav_blk1 bytes further.
      uint8_t* sav_dst = nullptr;
      long long sav_blk1 = 0;
      if constexpr (kSave) {
        const int word = *reinterpret_cast<const int*>(base_ptr + rec_off + sr * kRStage + hdr_off + 12);
        if constexpr (kX3) {
          sav_dst = p.sav + ((long long)((word >> 1) + (j & 1) * 2) << 13) + sav_row +
                    (uint32_t)(((4 * (word & 1) + (j >> 1)) ^ (r0 & 7)) << 4);
          sav_blk1 = (long long)(p.sav_np * 4) << 13;
        } else {
          sav_dst = p.sav + ((long long)word << 13) + sav_row + (uint32_t)((j ^ (r0 & 7)) << 4);
          sav_blk1 = (long long)(2 * p.sav_np) << 13;
        }
      }
#ifdef D2C_UNIT_TRACE
      const int trole = lane != 0 ? -1 : (warp == kGatherWarp0Fwd ? 3 : (warp == kGatherWarp0Fwd + 15 ? 4 : -1));
#define D2C_TG(e) do { if (trole >= 0) D2C_TR(trole, k, e); } while (0)
#else
#define D2C_TG(e) ((void)0)
#endif
      D2C_TG(0);
      issue(k, 1, c1);
      D2C_TG(1);
      if (!ptx::mbar_wait(a_empty(sa), ((k / kAStages) & 1) ^ 1, abort_flag)) break;
      D2C_TG(2);
      consume(k, 0, c0, sav_dst);
      D2C_TG(3);
      if (k + 1 < n_my_units) {
        if (!ptx::mbar_wait(r_full((k + 1) % kRStages), ((k + 1) / kRStages) & 1, abort_flag)) break;
        D2C_TG(4);
        issue(k + 1, 0, c0);
      }
      D2C_TG(5);
      consume(k, 1, c1, sav_dst + sav_blk1);
      D2C_TG(6);
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(a_full(sa));
        ptx::mbar_arrive(r_empty(sr));
      }
      D2C_TG(7);
    }
  }

  // ---- teardown ----
  ptx::tc_fence_before();
  __syncthreads();
#ifdef D2C_UNIT_TRACE
  if (p.trace && threadIdx.x == 0) {
    unsigned long long t1;
    unsigned smid;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    long long* rec = p.trace + 5 * 64 * 8 + blockIdx.x * 4;
    rec[0] = (long long)cta_t0; rec[1] = (long long)t1; rec[2] = (long long)smid; rec[3] = (long long)part_tab[32];
  }
#endif
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

