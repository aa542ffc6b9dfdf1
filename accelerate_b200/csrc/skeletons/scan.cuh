// scanl / scanl1 / scanl' / scanr / scanr1 / scanr' along the innermost dimension
// (Interpreter.hs:427-582) as ONE pass over the data: every tile publishes its
// aggregate, then looks back over its predecessors' descriptors (aggregate or
// inclusive prefix) to find its exclusive prefix, so each element is read once
// and written once (8 B/element for 4-byte types).
//
// Positions are handled in *logical* order q = 0..n-1: q = i for left scans and
// q = n-1-i for right scans, with the combination function flipped for right
// scans (out[i] = f x[i] out[i+1]).  The function need only be associative;
// operand order is preserved everywhere.
//
// Tiles are handed out by a ticket counter, so a tile's predecessors have
// always started before it: the look-back wait cannot deadlock.  It is bounded
// anyway: after `spin_limit` polls the kernel records ETIMEDOUT in the status
// word and leaves.
//
// Descriptors live in scratch memory and are tagged with a launch epoch, so
// they need no clearing between launches: status = epoch << 2 | state.
// SCAN_PACKED (one scalar leaf of at most 8 bytes): status and value share one
// 8- or 16-byte word that is written and read with a single access, so the
// look-back needs one L2 round trip per window and no fences.  Otherwise
// (tuples) the value is written first, then a fence, then the status word.
//
// Named parameters: n, rows, tiles_per_row, in_vec, out_vec, status, agg, incl,
// counter, epoch, err, spin_limit.
// ACC_SCAN_MODE: 0 inclusive (scanl1/scanr1); 1 seeded, n+1 results per row
// (scanl/scanr); 2 seeded, n results + row totals in a second array (scanl'/scanr').

#define SCAN_THREADS 256
#define SCAN_WARPS (SCAN_THREADS / 32)
#ifndef SCAN_ROUNDS
#define SCAN_ROUNDS 4
#endif
#define SCAN_WARP_ELEMS (SCAN_ROUNDS * 128)
#define SCAN_TILE (SCAN_WARPS * SCAN_WARP_ELEMS)
#ifndef SCAN_LOOK
#define SCAN_LOOK 2
#endif
#define SCAN_ST_AGG 1u
#define SCAN_ST_PREFIX 2u

#if ACC_SCAN2
#define ACC_SCAN_MODE 2
#elif ACC_SEEDED
#define ACC_SCAN_MODE 1
#else
#define ACC_SCAN_MODE 0
#endif

#ifndef SCAN_PACKED
#define SCAN_PACKED 0
#endif
// Barrier over the SCAN_THREADS threads that process tiles.  The ring kernel runs further
// warps (reducers, look-back) that must not take part, so it uses a named barrier instead.
#if defined(SCAN_RING) && SCAN_RING
#define SCAN_SYNC() asm volatile("bar.sync 1, %0;" ::"n"(SCAN_THREADS) : "memory")
#else
#define SCAN_SYNC() __syncthreads()
#endif
#ifndef SCAN_MIN_BLOCKS
#define SCAN_MIN_BLOCKS 1
#endif
// Descriptors of neighbouring tiles are polled by every CTA working near the front of the scan.
// Packed densely they share a few cache lines, i.e. one L2 slice serves all those polls; spread
// SCAN_DESC_STRIDE descriptors apart, they fall into different lines and slices.
#ifndef SCAN_DESC_STRIDE
#define SCAN_DESC_STRIDE 1
#endif
// pause after a look-back poll that found a predecessor not ready (polling harder only slows
// the stores being waited for)
#ifndef SCAN_BACKOFF_NS
#define SCAN_BACKOFF_NS 0
#endif
__device__ __forceinline__ void scan_backoff() {
#if SCAN_BACKOFF_NS > 0
  __nanosleep(SCAN_BACKOFF_NS);
#endif
}
#if SCAN_PACKED
#if SCAN_T_BYTES <= 4
// [63:32] status, [31:0] value bits
__device__ __forceinline__ void scan_desc_store(i64 base, i64 idx, u32 status, SCAN_T v) {
  u32 bits = 0;
  memcpy(&bits, &v, sizeof(SCAN_T));
  const u64 w = ((u64)status << 32) | bits;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(reinterpret_cast<u64*>(base) + idx * SCAN_DESC_STRIDE), "l"(w) : "memory");
}
__device__ __forceinline__ u32 scan_desc_load(i64 base, i64 idx, SCAN_T& v) {
  u64 w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(reinterpret_cast<const u64*>(base) + idx * SCAN_DESC_STRIDE) : "memory");
  const u32 bits = (u32)w;
  memcpy(&v, &bits, sizeof(SCAN_T));
  return (u32)(w >> 32);
}
#else
// 16-byte descriptor {value bits, status}: one aligned 128-bit access
__device__ __forceinline__ void scan_desc_store(i64 base, i64 idx, u32 status, SCAN_T v) {
  u64 bits = 0;
  memcpy(&bits, &v, sizeof(SCAN_T));
  asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(reinterpret_cast<ulonglong2*>(base) + idx * SCAN_DESC_STRIDE), "l"(bits), "l"((u64)status)
               : "memory");
}
__device__ __forceinline__ u32 scan_desc_load(i64 base, i64 idx, SCAN_T& v) {
  u64 bits, st;
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(bits), "=l"(st) : "l"(reinterpret_cast<const ulonglong2*>(base) + idx * SCAN_DESC_STRIDE) : "memory");
  memcpy(&v, &bits, sizeof(SCAN_T));
  return (u32)st;
}
#endif
#endif

// a . b with a earlier than b in logical order
__device__ __forceinline__ elt_t scan_op(const Params& p, const elt_t& a, const elt_t& b) {
#if ACC_RIGHT
  return F_combine(p, b, a);
#else
  return F_combine(p, a, b);
#endif
}
// a := a . b where either side may be absent
__device__ __forceinline__ void scan_join(const Params& p, elt_t& a, bool& ha, const elt_t& b, bool hb) {
  if (hb) {
    if (ha) a = scan_op(p, a, b);
    else { a = b; ha = true; }
  }
}
// a := b . a (b earlier)
__device__ __forceinline__ void scan_join_front(const Params& p, const elt_t& b, bool hb, elt_t& a, bool& ha) {
  if (hb) {
    if (ha) a = scan_op(p, b, a);
    else { a = b; ha = true; }
  }
}
template <class T> __device__ __forceinline__ T scan_ld_volatile(const T* src) {
  T r;
  if (sizeof(T) % 4 == 0) {
    const volatile u32* s = reinterpret_cast<const volatile u32*>(src);
    u32* d = reinterpret_cast<u32*>(&r);
    for (unsigned i = 0; i < sizeof(T) / 4; ++i) d[i] = s[i];
  } else {
    const volatile u8* s = reinterpret_cast<const volatile u8*>(src);
    u8* d = reinterpret_cast<u8*>(&r);
    for (unsigned i = 0; i < sizeof(T); ++i) d[i] = s[i];
  }
  return r;
}

// physical position of logical position q in the input row
__device__ __forceinline__ i64 scan_phys(i64 n, i64 q) {
#if ACC_RIGHT
  return n - 1 - q;
#else
  return q;
#endif
}

// Everything after the tile's elements are in registers: local scans, aggregate,
// look-back, per-thread prefixes, stores.  With GIVEN the caller already knows the tile's exclusive
// prefix (*given, if has_given): no descriptor is read or written.
template <bool FULL, bool GIVEN>
__device__ __forceinline__ void scan_tile_body(const Params& p, const i64 T, const i64 row, const i64 tt, elt_t (&item)[SCAN_ROUNDS][4],
                                               bool (&valid)[SCAN_ROUNDS][4], elt_t* sm_v, int* sm_h, elt_t* sm_excl, int* sm_flag,
                                               const elt_t* given, bool has_given) {
  const i64 n = p.n;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const i64 tile_q0 = tt * SCAN_TILE;
  const i64 warp_q0 = tile_q0 + (i64)warp * SCAN_WARP_ELEMS;
  const bool out_vec = p.out_vec != 0;
  elt_t tot[SCAN_ROUNDS];
  bool htot[SCAN_ROUNDS];
#pragma unroll
  for (int r = 0; r < SCAN_ROUNDS; ++r) {
    tot[r] = item[r][0];
    htot[r] = valid[r][0];
#pragma unroll
    for (int k = 1; k < 4; ++k) {
      if (valid[r][k]) {
        item[r][k] = scan_op(p, item[r][k - 1], item[r][k]);
        tot[r] = item[r][k];
      }
    }
  }
  // ---- warp-level inclusive scans of the per-thread totals, one per round ------
  elt_t lane_excl[SCAN_ROUNDS];
  bool hlane_excl[SCAN_ROUNDS];
  elt_t carry;           // rounds 0..r-1 of this warp
  bool hcarry = false;
  elt_t round_carry[SCAN_ROUNDS];
  bool hround_carry[SCAN_ROUNDS];
#pragma unroll
  for (int r = 0; r < SCAN_ROUNDS; ++r) {
    elt_t v = tot[r];
    bool h = htot[r];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const elt_t o = acc_shfl_up(v, d);
      const int oh = __shfl_up_sync(ACC_FULL_MASK, (int)h, d);
      if (lane >= d) scan_join_front(p, o, FULL || oh != 0, v, h);
    }
    const elt_t e = acc_shfl_up(v, 1);
    const int eh = __shfl_up_sync(ACC_FULL_MASK, (int)h, 1);
    lane_excl[r] = e;
    hlane_excl[r] = lane > 0 && (FULL || eh != 0);
    const elt_t rt = acc_shfl_idx(v, 31);
    const int rh = __shfl_sync(ACC_FULL_MASK, (int)h, 31);
    round_carry[r] = carry;
    hround_carry[r] = hcarry;
    scan_join(p, carry, hcarry, rt, FULL || rh != 0);
  }
  // carry now holds the warp's total
  if (lane == 0) { sm_v[warp] = carry; sm_h[warp] = hcarry; }
  SCAN_SYNC();

  // ---- tile aggregate, look-back (warp 0), tile exclusive prefix ---------------
  if (warp == 0) {
    elt_t agg;
    bool hagg = false;
#pragma unroll
    for (int w = 0; w < SCAN_WARPS; ++w) scan_join(p, agg, hagg, sm_v[w], sm_h[w] != 0);
    elt_t excl;
    bool hexcl = false;
    volatile u32* status = reinterpret_cast<volatile u32*>(p.status);
    elt_t* d_agg = reinterpret_cast<elt_t*>(p.agg);
    elt_t* d_incl = reinterpret_cast<elt_t*>(p.incl);
    const u32 epoch = (u32)p.epoch;
    int failed = 0;
    if (GIVEN) {
      if (has_given) { excl = *given; hexcl = true; }
    } else if (tt == 0) {
#if ACC_SEEDED
      excl = F_seed(p);
      hexcl = true;
#endif
    } else {
      if (lane == 0) {
        // an empty aggregate cannot occur: only the last tile of a row can be partial, and it has no successor
#if SCAN_PACKED
        scan_desc_store(p.status, T, (epoch << 2) | SCAN_ST_AGG, agg.l0);
#else
        d_agg[T] = agg;
        __threadfence();
        status[T] = (epoch << 2) | SCAN_ST_AGG;
#endif
      }
      const i64 row_first = T - tt;
      i64 look = T - 1;
      // Each lane inspects SCAN_LOOK consecutive predecessors per step (distance
      // SCAN_LOOK*lane + j from `look`), so one L2 round trip covers 32*SCAN_LOOK tiles: the
      // rate at which prefixes propagate, not bandwidth, is what limits a single-pass scan.
      for (;;) {
        u32 st[SCAN_LOOK];
        elt_t v[SCAN_LOOK];
        bool in[SCAN_LOOK], ready[SCAN_LOOK];
#pragma unroll
        for (int j = 0; j < SCAN_LOOK; ++j) {
          in[j] = look - (i64)(SCAN_LOOK * lane + j) >= row_first;
          ready[j] = !in[j];
          st[j] = 0;
        }
        for (i64 spins = 0;; ++spins) {
          bool all = true;
#pragma unroll
          for (int j = 0; j < SCAN_LOOK; ++j) {
            if (!ready[j]) {
              const i64 idx = look - (i64)(SCAN_LOOK * lane + j);
#if SCAN_PACKED
              st[j] = scan_desc_load(p.status, idx, v[j].l0);
#else
              st[j] = status[idx];
#endif
              ready[j] = (st[j] >> 2) == epoch;
              all = all && ready[j];
            }
          }
          if (all) break;
          if (spins > p.spin_limit) { failed = 1; break; }
          scan_backoff();
        }
        failed = __any_sync(ACC_FULL_MASK, failed);
        if (failed) break;
        // nearest inclusive prefix held by this lane (smallest j), if any
        int jp = SCAN_LOOK;
#pragma unroll
        for (int j = SCAN_LOOK - 1; j >= 0; --j)
          if (in[j] && (st[j] & 3u) == SCAN_ST_PREFIX) jp = j;
        const unsigned pm = __ballot_sync(ACC_FULL_MASK, jp < SCAN_LOOK);
        const int lstar = pm ? (__ffs((int)pm) - 1) : 32;
        // this lane's contribution: entries up to (and including) the nearest prefix, oldest first
        const int last = lane < lstar ? SCAN_LOOK - 1 : (lane == lstar ? jp : -1);
#if !SCAN_PACKED
        __threadfence();
#pragma unroll
        for (int j = 0; j < SCAN_LOOK; ++j)
          if (in[j] && j <= last) {
            const i64 idx = look - (i64)(SCAN_LOOK * lane + j);
            v[j] = scan_ld_volatile((st[j] & 3u) == SCAN_ST_PREFIX ? d_incl + idx : d_agg + idx);
          }
#endif
        elt_t c;
        bool hc = false;
#pragma unroll
        for (int j = SCAN_LOOK - 1; j >= 0; --j)
          if (in[j] && j <= last) scan_join(p, c, hc, v[j], true);
        // lane l holds older tiles than lane l-1
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const elt_t o = acc_shfl_down(c, d);
          const int oh = __shfl_down_sync(ACC_FULL_MASK, (int)hc, d);
          if (lane + d < 32) scan_join_front(p, o, oh != 0, c, hc);
        }
        scan_join_front(p, c, hc, excl, hexcl);  // meaningful in lane 0
        if (pm != 0 || look - 32 * SCAN_LOOK < row_first) break;
        look -= 32 * SCAN_LOOK;
      }
    }
    if (lane == 0) {
      if (failed) {
        acc_fail(p.err, 110 /* ETIMEDOUT */);
      } else {
        elt_t inc = excl;
        bool hinc = hexcl;
        scan_join(p, inc, hinc, agg, hagg);
        if (!GIVEN) {
#if SCAN_PACKED
          scan_desc_store(p.status, T, (epoch << 2) | SCAN_ST_PREFIX, inc.l0);
#else
          if (hinc) d_incl[T] = inc;
          __threadfence();
          status[T] = (epoch << 2) | SCAN_ST_PREFIX;
#endif
        }
#if ACC_SCAN_MODE != 0
        if (tt == p.tiles_per_row - 1) {
          // the row's total (seed included)
#if ACC_SCAN_MODE == 1
#if ACC_RIGHT
          OUT0_store(p, row * (n + 1), inc);
#else
          OUT0_store(p, row * (n + 1) + n, inc);
#endif
#else
          OUT1_store(p, row, inc);
#endif
        }
#endif
      }
      *sm_excl = excl;
      sm_flag[0] = hexcl ? 1 : 0;
      sm_flag[1] = failed;
    }
  }
  SCAN_SYNC();
  if (sm_flag[1]) return;

  // ---- per-thread prefixes and stores ----------------------------------------------
  elt_t base = *sm_excl;
  bool hbase = sm_flag[0] != 0;
  for (int w = 0; w < warp; ++w) scan_join(p, base, hbase, sm_v[w], sm_h[w] != 0);
#if ACC_SCAN_MODE == 1
  const i64 out_row = row * (n + 1);
#else
  const i64 out_row = row * n;
#endif
#pragma unroll
  for (int r = 0; r < SCAN_ROUNDS; ++r) {
    const i64 q = warp_q0 + r * 128 + lane * 4;
    elt_t pre = base;
    bool hpre = hbase;
    scan_join(p, pre, hpre, round_carry[r], hround_carry[r]);
    scan_join(p, pre, hpre, lane_excl[r], hlane_excl[r]);
    elt_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#if ACC_SCAN_MODE == 0
      o[k] = item[r][k];
      if (valid[r][k] && hpre) o[k] = scan_op(p, pre, item[r][k]);
#else
      // exclusive value: everything before position q+k (the seed guarantees it exists)
      if (k == 0) o[k] = pre;
      else if (valid[r][k - 1]) o[k] = scan_op(p, pre, item[r][k - 1]);
#endif
    }
    // where the four values go
#if ACC_SCAN_MODE == 1 && ACC_RIGHT
    const i64 pos0 = out_row + n - q;          // descending
#elif ACC_RIGHT
    const i64 pos0 = out_row + n - 1 - q;      // descending
#else
    const i64 pos0 = out_row + q;              // ascending
#endif
    if (FULL && out_vec) {
#if ACC_RIGHT
      elt_t w[4] = {o[3], o[2], o[1], o[0]};
      OUT0_store4(p, pos0 - 3, w);
#else
      OUT0_store4(p, pos0, o);
#endif
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (valid[r][k]) {
#if ACC_RIGHT
          OUT0_store(p, pos0 - k, o[k]);
#else
          OUT0_store(p, pos0 + k, o[k]);
#endif
        }
      }
    }
  }
}

template <bool FULL, bool GIVEN>
__device__ __forceinline__ void scan_tile(const Params& p, const i64 T, const i64 row, const i64 tt, elt_t* sm_v, int* sm_h,
                                          elt_t* sm_excl, int* sm_flag, const elt_t* given, bool has_given) {
  const i64 n = p.n;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const i64 tile_q0 = tt * SCAN_TILE;
  const i64 warp_q0 = tile_q0 + (i64)warp * SCAN_WARP_ELEMS;
  const bool in_vec = p.in_vec != 0;

  // ---- load; thread-local inclusive scan of each group of four ----------------
  elt_t item[SCAN_ROUNDS][4];
  bool valid[SCAN_ROUNDS][4];
#pragma unroll
  for (int r = 0; r < SCAN_ROUNDS; ++r) {
    const i64 q = warp_q0 + r * 128 + lane * 4;
    if (FULL && in_vec) {
#if ACC_RIGHT
      elt_t t4[4];
      D0_get4(p, row, n - 4 - q, t4);
#pragma unroll
      for (int k = 0; k < 4; ++k) item[r][k] = t4[3 - k];
#else
      D0_get4(p, row, q, item[r]);
#endif
#pragma unroll
      for (int k = 0; k < 4; ++k) valid[r][k] = true;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        valid[r][k] = FULL || (q + k < n);
        if (valid[r][k]) item[r][k] = D0_get(p, row, scan_phys(n, q + k));
      }
    }
  }
  scan_tile_body<FULL, GIVEN>(p, T, row, tt, item, valid, sm_v, sm_h, sm_excl, sm_flag, given, has_given);
}

extern "C" __global__ void __launch_bounds__(SCAN_THREADS, SCAN_MIN_BLOCKS) acc_scan(const Params p) {
  __shared__ elt_t sm_v[SCAN_WARPS];
  __shared__ int sm_h[SCAN_WARPS];
  __shared__ elt_t sm_excl;
  __shared__ int sm_flag[2];
  __shared__ unsigned sm_ticket;
  const i64 total_tiles = p.rows * p.tiles_per_row;
  if (threadIdx.x == 0) {
    unsigned* counter = reinterpret_cast<unsigned*>(p.counter);
    sm_ticket = atomicAdd(counter, 1u);
    if ((i64)sm_ticket == total_tiles - 1) *counter = 0u;  // every ticket has been handed out
  }
  __syncthreads();
  const i64 T = sm_ticket;
  const i64 row = T / p.tiles_per_row;
  const i64 tt = T - row * p.tiles_per_row;
  const bool full = (tt + 1) * SCAN_TILE <= p.n;
  if (full) scan_tile<true, false>(p, T, row, tt, sm_v, sm_h, &sm_excl, sm_flag, nullptr, false);
  else scan_tile<false, false>(p, T, row, tt, sm_v, sm_h, &sm_excl, sm_flag, nullptr, false);
}

// ---------------------------------------------------------------------------------
// acc_scan_ring: persistent CTAs that keep SCAN_SLOTS tiles each in a shared-memory
// ring.  A tile is bulk-copied in (cp.async.bulk + mbarrier); reducer warps publish
// its aggregate the moment it has arrived; a look-back warp finds its exclusive
// prefix.  The finisher warps take the oldest tile whose aggregate is out into
// registers, scan it there and hand its slot to the next ticket at once; they add the
// exclusive prefix and store when the look-back has delivered it.  A CTA therefore has
// SCAN_SLOTS tiles in shared memory plus one in registers in flight, and the look-back
// latency idles the memory system much less than in acc_scan, where a tile occupies
// registers from its load to its store.  Bookkeeping is per ring position (RING_META
// entries), separate from the data slots, because a slot is reused while the tile it
// held is still waiting for its prefix.
// Requirements (checked by the host): one scalar leaf (SCAN_PACKED), exactly one stream
// leaf of the same size, fast layout, in_vec and out_vec.  Partial tiles (the last of a
// row) are handled by scan_tile<false> inside the same kernel.
// Extra named parameters: total_tiles, total_batches, batches_per_row, gstatus, groups_per_row
// (`status` and `gstatus` hold one descriptor per batch and per group of batches).
// ---------------------------------------------------------------------------------
#if defined(SCAN_RING) && SCAN_RING
#ifndef SCAN_SLOTS
#define SCAN_SLOTS 6
#endif
#define RING_META (SCAN_SLOTS + 1)
#define RING_SLOT_BYTES (SCAN_TILE * SCAN_T_BYTES)
#define RING_GROUP (32 * SCAN_LOOK)
#define RING_PH_OWN 0
#define RING_PH_GROUPS 1
#define RING_PH_COMPUTE 2
#define RING_LOADING 0
#define RING_SCANNED 1
#define RING_RESOLVED 2
#define RING_DONE 3

__device__ __forceinline__ u32 ring_smem_addr(const void* ptr) { return (u32)__cvta_generic_to_shared(ptr); }
__device__ __forceinline__ void ring_mbar_init(u64* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ring_mbar_expect(u64* bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ring_smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ring_mbar_try_wait(u64* bar, u32 parity) {
  u32 ok;
  asm volatile(
      "{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(ok)
      : "r"(ring_smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void ring_bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ring_smem_addr(dst)), "l"(src),
               "r"(bytes), "r"(ring_smem_addr(bar))
               : "memory");
}
#define acc_bulk_g2s ring_bulk_g2s
extern __shared__ __align__(128) unsigned char scan_ring_smem[];

template <class T> __device__ __forceinline__ T ring_ldv(const T* p) { return *reinterpret_cast<const volatile T*>(p); }
template <class T> __device__ __forceinline__ void ring_stv(T* p, T v) { *reinterpret_cast<volatile T*>(p) = v; }

// Threads 0 .. SCAN_THREADS-1 (the workers) reduce arriving tiles and scan resolved tiles out of
// shared memory; SCAN_LB_WARPS further warps only run look-backs (ring position r is handled by
// warp r mod SCAN_LB_WARPS), so the look-back latency never stalls the workers.
#ifndef SCAN_LB_WARPS
#define SCAN_LB_WARPS 1
#endif
#ifndef RING_RED_WARPS
#define RING_RED_WARPS 2
#endif
#define RING_THREADS (SCAN_THREADS + 32 * RING_RED_WARPS + 32 * SCAN_LB_WARPS)
// state a tile must have reached before the finishers take it out of its slot: SCANNED (its
// aggregate is out; the default) or RESOLVED (its prefix is known: the tile then stays in its slot
// for the whole look-back)
#ifndef RING_GRAB_STATE
#define RING_GRAB_STATE RING_SCANNED
#endif
#define RING_ACT_SCAN 1
#define RING_ACT_FIN 2
#define RING_ACT_EXIT 4

// 8-byte elements: a lane's four results are 32 bytes, so a plain vector store per lane would write half a
// 32-byte sector per instruction.  The warp's 128 results of a round go through RING_STAGE_BYTES of shared memory
// per warp instead (written 32 bytes per lane, read back 16 bytes per lane from either half of the kilobyte),
// and every store instruction then covers 512 contiguous bytes.  `blk` is the first of the warp's 128 output
// elements, `mine` this lane's place in it (lane, or 31 - lane when the scan runs right to left).
// (Sending the staged kilobyte out with cp.async.bulk instead of reading it back was measured too: no faster for
// 8-byte elements, and slower than plain vector stores for 4-byte ones, 0.78 against 0.88 of the copy peak.)
#if SCAN_T_BYTES == 8
#define RING_STAGE_BYTES 1024
__device__ __forceinline__ void ring_store_block8(const Params& p, unsigned char* stage, i64 blk, int mine, const elt_t (&o)[4]) {
  const int lane = threadIdx.x & 31;
  uint4 lo, hi;
  memcpy(&lo.x, &o[0].l0, 8); memcpy(&lo.z, &o[1].l0, 8);
  memcpy(&hi.x, &o[2].l0, 8); memcpy(&hi.z, &o[3].l0, 8);
  uint4* mp = reinterpret_cast<uint4*>(stage + 32 * mine);
  const int h = (lane >> 2) & 1;                    // order of the halves alternates every four lanes (banks)
  mp[h] = h ? hi : lo;
  mp[h ^ 1] = h ? lo : hi;
  __syncwarp();
  const uint4 a = *reinterpret_cast<const uint4*>(stage + 16 * lane);
  const uint4 b = *reinterpret_cast<const uint4*>(stage + 512 + 16 * lane);
  __syncwarp();                                     // the staging kilobyte may be written again
  unsigned char* out = reinterpret_cast<unsigned char*>(p.out0_l0 + blk);
  *reinterpret_cast<uint4*>(out + 16 * lane) = a;
  *reinterpret_cast<uint4*>(out + 512 + 16 * lane) = b;
}
#else
#define RING_STAGE_BYTES 0
#endif

// The partial tile at the end of a row is rare and register-hungry: kept out of line so that it
// does not set the register budget of the common path.  Its exclusive prefix is handed in.
__device__ __noinline__ void ring_partial_tile(const Params& p, i64 T, i64 row, i64 tt, elt_t* sm_v, int* sm_h, elt_t* sm_excl, int* sm_flag,
                                               const elt_t* given, bool has_given) {
  scan_tile<false, true>(p, T, row, tt, sm_v, sm_h, sm_excl, sm_flag, given, has_given);
}

// Tickets hand out BATCHES of RING_BATCH consecutive tiles of a row.  Look-back descriptors
// describe batches: a CTA chains the tiles of its batch through shared memory (the exclusive
// prefix of tile j+1 is that of tile j combined with tile j's aggregate) and walks the global
// descriptors once per batch.  That divides the polling traffic and the number of descriptors by
// RING_BATCH; the price is that a batch's aggregate is published when its last tile has arrived.
#ifndef RING_BATCH
#define RING_BATCH SCAN_SLOTS
#endif
#define RING_VOID ((i64)-2)            // position past the last tile of its row (rows need not be whole batches)

extern "C" __global__ void __launch_bounds__(RING_THREADS, SCAN_MIN_BLOCKS) acc_scan_ring(const Params p) {
  __shared__ elt_t sm_v[SCAN_WARPS];
  __shared__ int sm_h[SCAN_WARPS];
  __shared__ elt_t sm_excl1;
  __shared__ int sm_flag1[2];
  __shared__ __align__(8) u64 full_bar[SCAN_SLOTS];
  // data slots: full_bar, slot_uses; ring positions (index pos % RING_META): everything else
  __shared__ i64 slot_tile[RING_META], slot_pos[RING_META], slot_batch[RING_META];
  __shared__ u32 slot_parity[RING_META], slot_uses[SCAN_SLOTS];
  __shared__ int slot_direct[RING_META], slot_state[RING_META], slot_hexcl[RING_META];
  __shared__ elt_t slot_agg[RING_META], slot_excl[RING_META];
  __shared__ int ctl_act, ctl_act2, sh_fail;   // thread 0's verdicts after the two waits of an iteration
  __shared__ i64 cur_batch;
  __shared__ elt_t red_v[2][RING_RED_WARPS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const i64 n = p.n;
  const i64 total_tiles = p.total_tiles;
  const i64 total_batches = p.total_batches;
  const u32 epoch = (u32)p.epoch;
  unsigned* counter = reinterpret_cast<unsigned*>(p.counter);
  unsigned* exits = counter + 1;

  // worker thread 0: the tile of ring position `pos` (tile pos % RING_BATCH of the CTA's current
  // batch; a new batch is drawn at every multiple of RING_BATCH); its data go to slot pos % SCAN_SLOTS
  auto fetch = [&](i64 pos) {
    const int s = (int)(pos % SCAN_SLOTS), m = (int)(pos % RING_META), j = (int)(pos % RING_BATCH);
    if (j == 0) cur_batch = (i64)atomicAdd(counter, 1u);
    const i64 K = cur_batch;
    i64 T = total_tiles;                                   // past the end: every role leaves its loop
    slot_batch[m] = K;
    slot_direct[m] = 1;
    slot_state[m] = RING_LOADING;
    if (K < total_batches) {
      const i64 row = K / p.batches_per_row;
      const i64 tt = (K - row * p.batches_per_row) * RING_BATCH + j;
      if (tt >= p.tiles_per_row) {
        T = RING_VOID;
      } else {
        T = row * p.tiles_per_row + tt;
        const i64 q0 = tt * SCAN_TILE;
        if (q0 + SCAN_TILE <= n) {
          slot_direct[m] = 0;
          slot_parity[m] = slot_uses[s] & 1u;
          slot_uses[s] += 1;
#if ACC_RIGHT
          const i64 src = row * n + (n - q0 - SCAN_TILE);
#else
          const i64 src = row * n + q0;
#endif
          unsigned char* base = scan_ring_smem + (size_t)s * RING_SLOT_BYTES;
          ring_mbar_expect(&full_bar[s], (u32)RING_SLOT_BYTES);
          D0_BULK_ISSUE(base, &full_bar[s], src)
        }
      }
    }
    slot_tile[m] = T;
    __threadfence_block();
    ring_stv(&slot_pos[m], pos);          // reducers and the look-back warp may now look at the entry
  };

  if (tid == 0) {
    for (int s = 0; s < SCAN_SLOTS; ++s) { ring_mbar_init(&full_bar[s], 1); slot_uses[s] = 0; }
    for (int m = 0; m < RING_META; ++m) { slot_pos[m] = -1; slot_tile[m] = total_tiles; slot_direct[m] = 1; slot_state[m] = RING_DONE; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    ctl_act = 0;
    ctl_act2 = 0;
    sh_fail = 0;
    cur_batch = total_batches;
  }
  __syncthreads();
  if (tid == 0)
    for (int s = 0; s < SCAN_SLOTS; ++s) fetch(s);
  __syncthreads();

  if (warp >= SCAN_WARPS + RING_RED_WARPS) {
    // ================= look-back warp ==================================================
    // One walk per batch, started as soon as the batch is drawn (its own data need not have
    // arrived).  Hierarchical: batches of a row are grouped by RING_GROUP.  Phase OWN reads the
    // earlier batches of the own group; phase GROUPS reads 32 group descriptors per step (aggregate
    // or inclusive prefix of a whole group); phase COMPUTE summarises a group nobody has summarised
    // yet from its batch descriptors and publishes the summary for every later walker.  The tiles of
    // the batch are then resolved in order from the batch's prefix and their aggregates.
    int lb_failed = 0;
    for (i64 r0 = 0; !lb_failed; r0 += RING_BATCH) {
      const int m0 = (int)(r0 % RING_META);
      i64 spins = 0;
      while (ring_ldv(&slot_pos[m0]) != r0) {
        if (++spins > p.spin_limit || ring_ldv(&sh_fail)) { lb_failed = 1; break; }
        __nanosleep(40);                             // leave the issue slots to the workers
      }
      if (lb_failed) break;
      __threadfence_block();
      const i64 K = slot_batch[m0];
      if (K >= total_batches) break;
      const i64 row = K / p.batches_per_row;
      const i64 kb = K - row * p.batches_per_row;
      const i64 row_first = K - kb;
      const i64 gid = kb / RING_GROUP;
      const i64 group_base = row * p.groups_per_row;
      elt_t excl;
      bool hexcl = false;
      int failed = 0;
      if (kb == 0) {
#if ACC_SEEDED
        excl = F_seed(p);
        hexcl = true;
#endif
      } else {
        int phase = (kb % RING_GROUP == 0) ? RING_PH_GROUPS : RING_PH_OWN;
        i64 g = gid - 1;
        i64 polls = 0;
        bool done = false;
        while (!done) {
          if (phase == RING_PH_GROUPS) {
            const i64 gi = g - lane;
            const bool in = gi >= 0;
            u32 st = 0;
            elt_t v;
            if (in) st = scan_desc_load(p.gstatus, group_base + gi, v.l0);
            const bool ready = in && (st >> 2) == epoch;
            const unsigned pm = __ballot_sync(ACC_FULL_MASK, ready && (st & 3u) == SCAN_ST_PREFIX);
            const unsigned em = __ballot_sync(ACC_FULL_MASK, in && !ready);
            const int lp = pm ? (__ffs((int)pm) - 1) : 32;
            const int lm = em ? (__ffs((int)em) - 1) : 32;
            elt_t c = v;
            bool hc = in && (lp < lm ? lane <= lp : lane < lm);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
              const elt_t o = acc_shfl_down(c, d);
              const int oh = __shfl_down_sync(ACC_FULL_MASK, (int)hc, d);
              if (lane + d < 32) scan_join_front(p, o, oh != 0, c, hc);
            }
            scan_join_front(p, c, hc, excl, hexcl);           // meaningful in lane 0
            if (lp < lm) done = true;
            else if (lm < 32) { g -= lm; phase = RING_PH_COMPUTE; }
            else { g -= 32; if (g < 0) done = true; }         // (group 0 is never a plain aggregate: not reached)
          } else {
            // batches hi, hi-1, ..., lo of the row (at most RING_GROUP = 32 * SCAN_LOOK of them)
            const i64 hi = phase == RING_PH_OWN ? kb - 1 : g * RING_GROUP + RING_GROUP - 1;
            const i64 lo = phase == RING_PH_OWN ? gid * RING_GROUP : g * RING_GROUP;
            u32 st[SCAN_LOOK];
            elt_t v[SCAN_LOOK];
            bool in[SCAN_LOOK], ready[SCAN_LOOK];
#pragma unroll
            for (int j = 0; j < SCAN_LOOK; ++j) {
              in[j] = hi - (i64)(SCAN_LOOK * lane + j) >= lo;
              ready[j] = !in[j];
              st[j] = 0;
            }
            for (;;) {                                  // entries found ready are not read again
              bool all = true;
#pragma unroll
              for (int j = 0; j < SCAN_LOOK; ++j)
                if (!ready[j]) {
                  st[j] = scan_desc_load(p.status, row_first + hi - (i64)(SCAN_LOOK * lane + j), v[j].l0);
                  ready[j] = (st[j] >> 2) == epoch;
                  all = all && ready[j];
                }
              if (__all_sync(ACC_FULL_MASK, all)) break;
              if (++polls > p.spin_limit || ring_ldv(&sh_fail)) { failed = 1; break; }
              scan_backoff();
            }
            if (failed) break;
            int jp = SCAN_LOOK;
#pragma unroll
            for (int j = SCAN_LOOK - 1; j >= 0; --j)
              if (in[j] && (st[j] & 3u) == SCAN_ST_PREFIX) jp = j;
            const unsigned pm = __ballot_sync(ACC_FULL_MASK, jp < SCAN_LOOK);
            const int lstar = pm ? (__ffs((int)pm) - 1) : 32;
            const int last = lane < lstar ? SCAN_LOOK - 1 : (lane == lstar ? jp : -1);
            elt_t c;
            bool hc = false;
#pragma unroll
            for (int j = SCAN_LOOK - 1; j >= 0; --j)
              if (in[j] && j <= last) scan_join(p, c, hc, v[j], true);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
              const elt_t o = acc_shfl_down(c, d);
              const int oh = __shfl_down_sync(ACC_FULL_MASK, (int)hc, d);
              if (lane + d < 32) scan_join_front(p, o, oh != 0, c, hc);
            }
            if (phase == RING_PH_COMPUTE && lane == 0 && hc)     // summary of group g, for every later walker
              scan_desc_store(p.gstatus, group_base + g, (epoch << 2) | (pm ? SCAN_ST_PREFIX : SCAN_ST_AGG), c.l0);
            scan_join_front(p, c, hc, excl, hexcl);             // meaningful in lane 0
            if (pm != 0) done = true;
            else {
              g = (phase == RING_PH_OWN) ? gid - 1 : g - 1;
              phase = RING_PH_GROUPS;
              if (g < 0) done = true;                           // start of the row reached
            }
          }
        }
      }
      if (failed) { lb_failed = 1; break; }
      // resolve the batch's tiles in order (lane 0 holds the running prefix)
      bool whole = true;                                         // all RING_BATCH tiles present and full
      for (int j = 0; j < RING_BATCH; ++j) {
        const i64 r = r0 + j;
        const int m = (int)(r % RING_META);
        spins = 0;
        while (ring_ldv(&slot_pos[m]) != r) {
          if (++spins > p.spin_limit || ring_ldv(&sh_fail)) { failed = 1; break; }
          __nanosleep(40);
        }
        if (failed) break;
        __threadfence_block();
        const i64 T = slot_tile[m];
        if (T == RING_VOID) { whole = false; break; }             // the row ended inside this batch
        if (slot_direct[m]) {
          // partial tile, the last of its row: the finishers scan it from global memory with this prefix
          if (lane == 0) {
            slot_excl[m] = excl;
            slot_hexcl[m] = hexcl ? 1 : 0;
            __threadfence_block();
            ring_stv(&slot_state[m], RING_RESOLVED);
          }
          whole = false;
          break;
        }
        spins = 0;
        while (ring_ldv(&slot_state[m]) < RING_SCANNED) {
          if (++spins > p.spin_limit || ring_ldv(&sh_fail)) { failed = 1; break; }
          __nanosleep(40);
        }
        if (failed) break;
        __threadfence_block();
        if (lane == 0) {
          const elt_t agg = slot_agg[m];
          slot_excl[m] = excl;
          slot_hexcl[m] = hexcl ? 1 : 0;
          __threadfence_block();
          ring_stv(&slot_state[m], RING_RESOLVED);
          scan_join(p, excl, hexcl, agg, true);                   // prefix of the next tile
        }
        __syncwarp();
      }
      if (failed) { lb_failed = 1; break; }
      if (whole && lane == 0) {
        // excl is now the inclusive prefix of the whole batch
        scan_desc_store(p.status, K, (epoch << 2) | SCAN_ST_PREFIX, excl.l0);
        if ((kb % RING_GROUP) == RING_GROUP - 1)                  // also the inclusive prefix of its whole group
          scan_desc_store(p.gstatus, group_base + gid, (epoch << 2) | SCAN_ST_PREFIX, excl.l0);
      }
      __syncwarp();
    }
    // a wait gave up: tell the workers (the flag may also have been raised by them)
    if (lb_failed && lane == 0) ring_stv(&sh_fail, 1);
  } else if (warp >= SCAN_WARPS) {
    // ================= reducers ========================================================
    // Every later batch of the row waits for this batch's aggregate, so tile aggregates are computed
    // by warps that do nothing else, the moment the data has arrived; the scan itself is left to
    // the finishers.  The batch's aggregate is published with its last tile.
    const int rt = tid - SCAN_THREADS, rw = warp - SCAN_WARPS;
    int red_failed = 0;
    elt_t bacc;                                      // thread rt == 0: aggregate of the batch so far
    for (i64 r = 0;; ++r) {
      const int s = (int)(r % RING_META), ds = (int)(r % SCAN_SLOTS), j = (int)(r % RING_BATCH);
      i64 spins = 0;
      while (ring_ldv(&slot_pos[s]) != r) {
        if (++spins > p.spin_limit || ring_ldv(&sh_fail)) { red_failed = 1; break; }
        __nanosleep(40);
      }
      if (red_failed) break;
      __threadfence_block();
      const i64 T = slot_tile[s];
      if (T >= total_tiles) break;
      if (T == RING_VOID || slot_direct[s]) continue;           // nothing to reduce: the row ends here, nobody needs this batch's aggregate
      spins = 0;
      while (!ring_mbar_try_wait(&full_bar[ds], slot_parity[s])) {
        if (++spins > p.spin_limit || ring_ldv(&sh_fail)) { red_failed = 1; break; }
      }
      if (red_failed) break;
      const i64 row = T / p.tiles_per_row;
      const i64 tt = T - row * p.tiles_per_row;
      const unsigned char* base = scan_ring_smem + (size_t)ds * RING_SLOT_BYTES;
      // warp rw reduces elements [rw, rw + 1) * SCAN_TILE / RING_RED_WARPS in rounds of 128
      constexpr int RED_ROUNDS = SCAN_TILE / (128 * RING_RED_WARPS);
      elt_t tot;
#if ACC_COMMUTATIVE
      // lanes accumulate their own quads across rounds; one warp reduction at the end
#pragma unroll 4
      for (int k = 0; k < RED_ROUNDS; ++k) {
        const int e = (rw * RED_ROUNDS + k) * 128 + lane * 4;
        const i64 q = tt * SCAN_TILE + e;
        elt_t t4[4];
#if ACC_RIGHT
        D0_get4_sm(p, row, n - 4 - q, base, SCAN_TILE - 4 - e, t4);
#else
        D0_get4_sm(p, row, q, base, e, t4);
#endif
        const elt_t v = scan_op(p, scan_op(p, t4[0], t4[1]), scan_op(p, t4[2], t4[3]));
        if (k == 0) tot = v;
        else tot = scan_op(p, tot, v);
      }
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) tot = scan_op(p, tot, acc_shfl_down(tot, d));
#else
#pragma unroll 2
      for (int k = 0; k < RED_ROUNDS; ++k) {
        const int e = (rw * RED_ROUNDS + k) * 128 + lane * 4;
        const i64 q = tt * SCAN_TILE + e;
        elt_t t4[4];
#if ACC_RIGHT
        D0_get4_sm(p, row, n - 4 - q, base, SCAN_TILE - 4 - e, t4);
        elt_t v = scan_op(p, scan_op(p, scan_op(p, t4[3], t4[2]), t4[1]), t4[0]);
#else
        D0_get4_sm(p, row, q, base, e, t4);
        elt_t v = scan_op(p, scan_op(p, scan_op(p, t4[0], t4[1]), t4[2]), t4[3]);
#endif
        // lanes in order within the round, rounds in order within the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const elt_t o = acc_shfl_down(v, d);
          if (lane + d < 32) v = scan_op(p, v, o);
        }
        if (k == 0) tot = v;
        else tot = scan_op(p, tot, v);
      }
#endif
      if (lane == 0) red_v[r & 1][rw] = tot;
      asm volatile("bar.sync 2, %0;" ::"n"(32 * RING_RED_WARPS) : "memory");
      if (rt == 0) {
        elt_t agg = red_v[r & 1][0];
        for (int w = 1; w < RING_RED_WARPS; ++w) agg = scan_op(p, agg, red_v[r & 1][w]);
        const i64 K = slot_batch[s];     // (read before the state change below lets the entry move on)
        slot_agg[s] = agg;
        __threadfence_block();
        ring_stv(&slot_state[s], RING_SCANNED);
        if (j == 0) bacc = agg;
        else bacc = scan_op(p, bacc, agg);
        if (j == RING_BATCH - 1) {
          // the batch is complete (a batch cut short by the end of its row has no successor)
          if (K % p.batches_per_row == 0) {
#if ACC_SEEDED
            scan_desc_store(p.status, K, (epoch << 2) | SCAN_ST_PREFIX, scan_op(p, F_seed(p), bacc).l0);
#else
            scan_desc_store(p.status, K, (epoch << 2) | SCAN_ST_PREFIX, bacc.l0);
#endif
          } else {
            scan_desc_store(p.status, K, (epoch << 2) | SCAN_ST_AGG, bacc.l0);
          }
        }
      }
    }
    if (red_failed && lane == 0) ring_stv(&sh_fail, 1);
  } else {
    // ================= finishers ========================================================
    // Ring positions are finished in order.  As soon as the tile's aggregate is out (the reducers
    // are done with the slot) the tile is read into registers and scanned there, and its slot is
    // handed to the next tile; prefix and stores follow when the look-back warp has resolved the tile.
    i64 idle = 0;                          // thread 0: consecutive polls without anything to do
#if SCAN_T_BYTES == 8
    unsigned char* stage = scan_ring_smem + (size_t)SCAN_SLOTS * RING_SLOT_BYTES + (size_t)warp * RING_STAGE_BYTES;
#endif
    for (i64 r = 0;; ++r) {
      const int fs = (int)(r % SCAN_SLOTS), fm = (int)(r % RING_META);
      const i64 T = slot_tile[fm];         // written by thread 0 before a SCAN_SYNC
      if (T >= total_tiles) break;
      if (T == RING_VOID) {
        SCAN_SYNC();
        if (tid == 0) fetch(r + SCAN_SLOTS);
        SCAN_SYNC();
        continue;
      }
      const i64 row = T / p.tiles_per_row;
      const i64 tt = T - row * p.tiles_per_row;
      if (slot_direct[fm]) {
        // partial tile: wait for its prefix, then start to finish from global memory
        if (tid == 0) {
          idle = 0;
          while (ring_ldv(&slot_state[fm]) < RING_RESOLVED) {
            if (++idle > p.spin_limit) ring_stv(&sh_fail, 1);
            if (ring_ldv(&sh_fail)) break;
            __nanosleep(40);
          }
          ctl_act = ring_ldv(&sh_fail) ? RING_ACT_EXIT : RING_ACT_FIN;
        }
        SCAN_SYNC();
        if (ctl_act == RING_ACT_EXIT) break;
        const elt_t gexcl = slot_excl[fm];
        ring_partial_tile(p, T, row, tt, sm_v, sm_h, &sm_excl1, sm_flag1, &gexcl, slot_hexcl[fm] != 0);
        SCAN_SYNC();
        if (tid == 0) fetch(r + SCAN_SLOTS);
        SCAN_SYNC();                     // the next tile of this slot is known to every finisher
      } else {
        if (tid == 0) {
          idle = 0;
          while (ring_ldv(&slot_state[fm]) < RING_GRAB_STATE) {
            if (++idle > p.spin_limit) ring_stv(&sh_fail, 1);     // the aggregate never arrived: give up
            if (ring_ldv(&sh_fail)) break;
            __nanosleep(40);
          }
          ctl_act = ring_ldv(&sh_fail) ? RING_ACT_EXIT : RING_ACT_FIN;
        }
        SCAN_SYNC();
        if (ctl_act == RING_ACT_EXIT) break;
        // (the data was seen complete by the reducers, whose state change this thread observed
        // through thread 0 and the barrier; testing the barrier again costs nothing and makes the
        // bulk copy's writes visible to this thread in its own right)
        ring_mbar_try_wait(&full_bar[fs], slot_parity[fm]);
        const unsigned char* base = scan_ring_smem + (size_t)fs * RING_SLOT_BYTES;
#if ACC_SCAN_MODE == 1
        const i64 out_row = row * (n + 1);
#else
        const i64 out_row = row * n;
#endif
        const i64 warp_q0 = tt * SCAN_TILE + (i64)warp * SCAN_WARP_ELEMS;
        elt_t item[SCAN_ROUNDS][4];
#pragma unroll
        for (int r2 = 0; r2 < SCAN_ROUNDS; ++r2) {
          const int e = warp * SCAN_WARP_ELEMS + r2 * 128 + lane * 4;
          const i64 q = warp_q0 + r2 * 128 + lane * 4;
#if ACC_RIGHT
          elt_t t4[4];
          D0_get4_sm(p, row, n - 4 - q, base, SCAN_TILE - 4 - e, t4);
#pragma unroll
          for (int k = 0; k < 4; ++k) item[r2][k] = t4[3 - k];
#else
          D0_get4_sm(p, row, q, base, e, item[r2]);
#endif
#pragma unroll
          for (int k = 1; k < 4; ++k) item[r2][k] = scan_op(p, item[r2][k - 1], item[r2][k]);
        }
        elt_t lane_excl[SCAN_ROUNDS], round_carry[SCAN_ROUNDS];
        elt_t carry;
#pragma unroll
        for (int r2 = 0; r2 < SCAN_ROUNDS; ++r2) {
          elt_t v = item[r2][3];
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            const elt_t o = acc_shfl_up(v, d);
            if (lane >= d) v = scan_op(p, o, v);
          }
          lane_excl[r2] = acc_shfl_up(v, 1);
          const elt_t rtot = acc_shfl_idx(v, 31);
          round_carry[r2] = carry;
          if (r2 == 0) carry = rtot;
          else carry = scan_op(p, carry, rtot);
        }
        if (lane == 0) sm_v[warp] = carry;
        SCAN_SYNC();                     // every finisher has the slot's data in registers
        if (tid == 0) {
          fetch(r + SCAN_SLOTS);         // the slot takes the next tile while this one waits for its prefix
          idle = 0;
          while (ring_ldv(&slot_state[fm]) < RING_RESOLVED) {
            if (++idle > p.spin_limit) ring_stv(&sh_fail, 1);     // the prefix never arrived: give up
            if (ring_ldv(&sh_fail)) break;
            __nanosleep(20);
          }
          ctl_act2 = ring_ldv(&sh_fail) ? RING_ACT_EXIT : RING_ACT_FIN;
        }
        SCAN_SYNC();
        if (ctl_act2 == RING_ACT_EXIT) break;
        const elt_t excl = slot_excl[fm];
        const bool hexcl = slot_hexcl[fm] != 0;
        elt_t wbase = excl;             // everything before this warp's part: tile prefix, then earlier warps
        bool hwb = hexcl;
        for (int w = 0; w < warp; ++w) scan_join(p, wbase, hwb, sm_v[w], true);
#pragma unroll
        for (int r2 = 0; r2 < SCAN_ROUNDS; ++r2) {
          const int e = warp * SCAN_WARP_ELEMS + r2 * 128 + lane * 4;
          const i64 q = tt * SCAN_TILE + e;
          elt_t pre = wbase;
          bool hpre = hwb;
          scan_join(p, pre, hpre, round_carry[r2], r2 > 0);
          scan_join(p, pre, hpre, lane_excl[r2], lane > 0);
          elt_t o[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
#if ACC_SCAN_MODE == 0
            o[k] = hpre ? scan_op(p, pre, item[r2][k]) : item[r2][k];
#else
            if (k == 0) o[k] = pre;                                // the seed guarantees a prefix exists
            else o[k] = scan_op(p, pre, item[r2][k - 1]);
#endif
          }
#if ACC_SCAN_MODE == 1 && ACC_RIGHT
          const i64 pos0 = out_row + n - q;
#elif ACC_RIGHT
          const i64 pos0 = out_row + n - 1 - q;
#else
          const i64 pos0 = out_row + q;
#endif
#if ACC_RIGHT
          elt_t w4[4] = {o[3], o[2], o[1], o[0]};
#if SCAN_T_BYTES == 8
          ring_store_block8(p, stage, pos0 - 3 - 4 * (31 - lane), 31 - lane, w4);
#else
          OUT0_store4(p, pos0 - 3, w4);
#endif
#elif SCAN_T_BYTES == 8
          ring_store_block8(p, stage, pos0 - 4 * lane, lane, o);
#else
          OUT0_store4(p, pos0, o);
#endif
        }
#if ACC_SCAN_MODE != 0
        if (tid == 0 && tt == p.tiles_per_row - 1) {
          const elt_t tot = scan_op(p, excl, slot_agg[fm]);
#if ACC_SCAN_MODE == 1
#if ACC_RIGHT
          OUT0_store(p, row * (n + 1), tot);
#else
          OUT0_store(p, row * (n + 1) + n, tot);
#endif
#else
          OUT1_store(p, row, tot);
#endif
        }
#endif
        // (sm_v, ctl_act and this entry's bookkeeping are next written after the barriers of
        // the following iteration, which every finisher reaches only after its reads above)
      }
    }
  }
  // everybody meets here; the look-back warp leaves its loop when it sees a batch past the end,
  // a failure flag, or an expired wait (in which case it raises the flag itself)
  __syncthreads();
  if (tid == 0) {
    // Wait for bulk copies still in flight into this CTA's shared memory (only after a failure can
    // there be any).  A bulk copy completes without the help of any other CTA, so this wait gets a
    // bound of its own, far above the time a copy can take.
    for (int m = 0; m < RING_META; ++m) {
      if (slot_pos[m] >= 0 && slot_tile[m] >= 0 && slot_tile[m] < total_tiles && !slot_direct[m] && slot_state[m] == RING_LOADING) {
        i64 spins = 0;
        while (!ring_mbar_try_wait(&full_bar[slot_pos[m] % SCAN_SLOTS], slot_parity[m]))
          if (++spins > ((i64)1 << 26)) break;
      }
    }
    if (sh_fail) acc_fail(p.err, 110 /* ETIMEDOUT */);
    __threadfence();
    if (atomicAdd(exits, 1u) == gridDim.x - 1) { *counter = 0u; *exits = 0u; }
  }
}
#endif
