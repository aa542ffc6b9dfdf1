// stencil / stencil2 on rank-2 arrays (Interpreter.hs:637-839) without shared
// memory.  A warp loads a strip of 128 columns (four per lane, one 128-bit load
// per input row) and produces the 120 columns of lanes 1..30; lanes 0 and 31
// only supply the halo columns (stencil radius <= 4) to their neighbours, so
// neighbouring strips overlap by eight columns (re-read from L1/L2) and no lane
// ever issues a separate halo load.  The warp marches down ST2_ROWS rows.
//
// Each thread keeps a window of input rows of its columns in registers: the
// 2*ry+1 rows the current output row needs plus ST2_DEPTH rows requested ahead
// (loads land directly in their window slot, so several rows per warp are in
// flight).  The rx columns to either side come from the neighbouring lanes by
// warp shuffle just before a row is first used.  Out-of-range rows are
// redirected to the row the boundary condition names (clamp, mirror, wrap), so
// they keep the vector path; out-of-range columns (first and last strip only),
// Constant/Function boundaries and delayed inputs are evaluated element by
// element (ST_bounded, Interpreter.hs:797-839).
// HBM traffic: one read per input point and one write per output point, plus
// 2*ry halo rows per ST2_ROWS rows.
//
// Named parameters: o1, o2 (output rows, columns), row0, row1 (the rows to produce: all of them, or a
// window of an existing output array), tiles1 (row blocks of the window), tiles2 (strips of 120
// output columns), vec (o2 % 4 == 0, 16-byte aligned output); with ST2_FRAME also fr_strips, fr_r0, fr_r1 (see the kernel).
// One warp per task: grid = ceil(tiles1 * tiles2 / ST2_WARPS).

#ifndef ST2_BULK
#define ST2_BULK 0
#endif
#ifndef ST2_FRAME
#define ST2_FRAME 0      // 1: the kernel computes the frame around acc_stencil2d_bulk's part (see the kernel)
#endif
#ifndef ST2_TWOWIN
#define ST2_TWOWIN 0     // 1: two row ranges (named parameters row2, row3 besides row0, row1)
#endif
#ifndef ST2_WARPS
#define ST2_WARPS 4
#endif
#ifndef ST2_ROWS
#define ST2_ROWS 32
#endif
#ifndef ST2_MIN_BLOCKS
#define ST2_MIN_BLOCKS 1
#endif
#define ST2_THREADS (ST2_WARPS * 32)
#define ST2_STRIP 120
#define ST2_AHEAD (2 * ST_RYMAX + ST2_DEPTH)   // rows requested before the first output row

#if !ST2_BULK
#define ST2_PROLOGUE(D)                                                   \
  if ((D) < ST2_AHEAD) { ST2_ISSUE_ALL((D) % ST_HW, y0 - ST_RYMAX + (D)) }
#define ST2_PROLOGUE_COMMIT(D)                                            \
  if ((D) < 2 * ST_RYMAX) { ST2_COMMIT_ALL((D) % ST_HW) }

#define ST2_STEP(PH)                                                                   \
  if ((PH) < ST_HW && y + (PH) < y1) {                                                 \
    const int yy = y + (PH);                                                           \
    if (yy + ST2_DEPTH < y1) { ST2_ISSUE_ALL(((PH) + ST_HW - 1) % ST_HW, yy + ST_RYMAX + ST2_DEPTH) } \
    ST2_COMMIT_ALL(((PH) + 2 * ST_RYMAX) % ST_HW)                                      \
    if (writer) {                                                                      \
      elt_t o[4];                                                                      \
      o[0] = ST2_apply<0, (PH) % ST_HW>(p, ST2_WIN_ARGS);                              \
      o[1] = ST2_apply<1, (PH) % ST_HW>(p, ST2_WIN_ARGS);                              \
      o[2] = ST2_apply<2, (PH) % ST_HW>(p, ST2_WIN_ARGS);                              \
      o[3] = ST2_apply<3, (PH) % ST_HW>(p, ST2_WIN_ARGS);                              \
      const i64 lin = (i64)yy * (i64)o2 + (i64)gx0;                                    \
      if (st_vec) {                                                                    \
        OUT0_store4(p, lin, o);                                                        \
      } else {                                                                         \
        _Pragma("unroll") for (int k = 0; k < 4; ++k)                                  \
          if (gx0 + k < o2) OUT0_store(p, lin + k, o[k]);                              \
      }                                                                                \
    }                                                                                  \
  }

// The same step for a warp whose rows all lie inside the arrays and whose lanes are all on the
// vector path: no row redirection, no range checks, one predicated vector store.
#define ST2_FSTEP(PH)                                                                  \
  if ((PH) < ST_HW) {                                                                  \
    const int yy = y + (PH);                                                           \
    ST2_ISSUE_ALL_FAST(((PH) + ST_HW - 1) % ST_HW, yy + ST_RYMAX + ST2_DEPTH)          \
    ST2_COMMIT_ALL(((PH) + 2 * ST_RYMAX) % ST_HW)                                      \
    elt_t o[4];                                                                        \
    o[0] = ST2_apply<0, (PH) % ST_HW>(p, ST2_WIN_ARGS);                                \
    o[1] = ST2_apply<1, (PH) % ST_HW>(p, ST2_WIN_ARGS);                                \
    o[2] = ST2_apply<2, (PH) % ST_HW>(p, ST2_WIN_ARGS);                                \
    o[3] = ST2_apply<3, (PH) % ST_HW>(p, ST2_WIN_ARGS);                                \
    if (writer) OUT0_store4(p, (i64)yy * (i64)o2 + (i64)gx0, o);                       \
  }

extern "C" __global__ void __launch_bounds__(ST2_THREADS, ST2_MIN_BLOCKS) acc_stencil2d(const Params p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#if ST2_TWOWIN
  // two row ranges in one launch: rows row0 .. row1-1, then rows row2 .. row3-1 (tiles1 counts the row blocks of both)
  const i64 task = (i64)blockIdx.x * ST2_WARPS + warp;
  if (task >= p.tiles1 * p.tiles2) return;
  const int o1 = (int)p.o1, o2 = (int)p.o2;
  const int rb = (int)(task / p.tiles2);
  const int strip = (int)(task - (i64)rb * p.tiles2);
  const int gx0 = strip * ST2_STRIP - 4 + lane * 4;
  const int rb1 = (int)((p.row1 - p.row0 + ST2_ROWS - 1) / ST2_ROWS);
  const int y0 = rb < rb1 ? (int)p.row0 + rb * ST2_ROWS : (int)p.row2 + (rb - rb1) * ST2_ROWS;
  const int y1 = min(y0 + ST2_ROWS, rb < rb1 ? (int)p.row1 : (int)p.row3);
#elif !ST2_FRAME
  const i64 ntasks = p.tiles1 * p.tiles2;
  const i64 task = (i64)blockIdx.x * ST2_WARPS + warp;
  if (task >= ntasks) return;
  const int o1 = (int)p.o1, o2 = (int)p.o2;
  const int rb = (int)(task / p.tiles2);
  const int strip = (int)(task - (i64)rb * p.tiles2);
  const int gx0 = strip * ST2_STRIP - 4 + lane * 4;
  const int y0 = (int)p.row0 + rb * ST2_ROWS;
  const int y1 = min(y0 + ST2_ROWS, (int)p.row1);
#else
  const i64 task = (i64)blockIdx.x * ST2_WARPS + warp;
  const int o1 = (int)p.o1, o2 = (int)p.o2;
  int strip, y0, y1;
  {
    // The frame around the part acc_stencil2d_bulk computes (strips 1 .. fr_strips, rows fr_r0 .. fr_r1-1):
    // region A, strip 0 and the strips after fr_strips over every row; region C, the rows above fr_r0 of
    // the middle strips; region D, the rows from fr_r1 on of the middle strips.  tiles2 counts all strips.
    const i64 sin = p.fr_strips, ca = p.tiles2 - sin;
    const i64 ra = (o1 + ST2_ROWS - 1) / ST2_ROWS, rc = (p.fr_r0 + ST2_ROWS - 1) / ST2_ROWS, rd = (o1 - p.fr_r1 + ST2_ROWS - 1) / ST2_ROWS;
    const i64 na = ca * ra, nc = sin * rc, nd = sin * rd;
    int ylim;
    if (task < na) {
      const i64 c = task % ca;
      strip = (int)(c == 0 ? 0 : sin + c);
      y0 = (int)(task / ca) * ST2_ROWS;
      ylim = o1;
    } else if (task < na + nc) {
      const i64 t = task - na;
      strip = 1 + (int)(t % sin);
      y0 = (int)(t / sin) * ST2_ROWS;
      ylim = (int)p.fr_r0;
    } else if (task < na + nc + nd) {
      const i64 t = task - na - nc;
      strip = 1 + (int)(t % sin);
      y0 = (int)p.fr_r1 + (int)(t / sin) * ST2_ROWS;
      ylim = o1;
    } else {
      return;
    }
    y1 = min(y0 + ST2_ROWS, ylim);
  }
  const int gx0 = strip * ST2_STRIP - 4 + lane * 4;
#endif
  (void)o1;
  // lanes 1..30 produce output; the strip's columns beyond the array produce none
  const bool writer = lane >= 1 && lane <= 30 && gx0 < o2;
  const bool st_vec = p.vec != 0 && gx0 + 4 <= o2;
  ST2_LANE_FAST_DECL
  ST2_WIN_DECL
  // rows y0-ry .. y0+ry+depth-1 go to slots 0 .. 2*ry+depth-1 (at most 8+8 of them)
  ST2_PROLOGUE(0) ST2_PROLOGUE(1) ST2_PROLOGUE(2) ST2_PROLOGUE(3) ST2_PROLOGUE(4) ST2_PROLOGUE(5) ST2_PROLOGUE(6) ST2_PROLOGUE(7)
  ST2_PROLOGUE(8) ST2_PROLOGUE(9) ST2_PROLOGUE(10) ST2_PROLOGUE(11) ST2_PROLOGUE(12) ST2_PROLOGUE(13) ST2_PROLOGUE(14) ST2_PROLOGUE(15)
  ST2_PROLOGUE_COMMIT(0) ST2_PROLOGUE_COMMIT(1) ST2_PROLOGUE_COMMIT(2) ST2_PROLOGUE_COMMIT(3)
  ST2_PROLOGUE_COMMIT(4) ST2_PROLOGUE_COMMIT(5) ST2_PROLOGUE_COMMIT(6) ST2_PROLOGUE_COMMIT(7)
  int y = y0;
  // rows y0-ry .. y1+ry+depth-1 inside every input, every lane on the vector path (interior strips)
  const bool interior = __all_sync(ACC_FULL_MASK, ST2_ALL_LANE_FAST && (st_vec || !writer)) && y0 - ST_RYMAX >= 0 &&
                        y1 + ST_RYMAX + ST2_DEPTH <= ST2_MIN_E0;
  if (interior) {
    for (; y + ST_HW <= y1; y += ST_HW) {
      ST2_FSTEP(0) ST2_FSTEP(1) ST2_FSTEP(2) ST2_FSTEP(3) ST2_FSTEP(4) ST2_FSTEP(5) ST2_FSTEP(6) ST2_FSTEP(7)
      ST2_FSTEP(8) ST2_FSTEP(9) ST2_FSTEP(10) ST2_FSTEP(11) ST2_FSTEP(12) ST2_FSTEP(13) ST2_FSTEP(14) ST2_FSTEP(15) ST2_FSTEP(16)
    }
  }
  for (; y < y1; y += ST_HW) {
    ST2_STEP(0) ST2_STEP(1) ST2_STEP(2) ST2_STEP(3) ST2_STEP(4) ST2_STEP(5) ST2_STEP(6) ST2_STEP(7)
    ST2_STEP(8) ST2_STEP(9) ST2_STEP(10) ST2_STEP(11) ST2_STEP(12) ST2_STEP(13) ST2_STEP(14) ST2_STEP(15) ST2_STEP(16)
  }
}

#endif

#if ST2_BULK
// ---------------------------------------------------------------------------------
// acc_stencil2d_bulk: the same computation with the input rows staged through shared
// memory.  In acc_stencil2d the rows requested ahead live in registers, which caps what
// a warp can have in flight (two inputs of 3x3 taps already cost 150 registers for four
// rows ahead).  Here every warp owns a ring of ST2B_SLOTS row slots in shared memory; one
// lane keeps the ring full with bulk copies (cp.async.bulk, one per stream leaf and row:
// the strip's 128 columns, completion counted by the slot's mbarrier), and the warp
// takes a row out of its slot into the register window (ST_H rows, nothing ahead) when
// the row is first needed.  Warps do not synchronise with one another.
// Only tasks whose 128 columns and ST_H-1 halo rows lie inside every input are handled
// (strips strip0 .. strip0+tiles2-1, rows row0 .. row1-1, in blocks of ST2B_ROWS); the
// frame around them is left to acc_stencil2d.  Requires ST2_BULK_OK (every input read
// through streams with leaves of 4 or 8 bytes), the fast layout, row lengths that are
// multiples of 4 and a vector-aligned output; compiled with ST2_DEPTH 0 and SCAN_TILE 128.
// Extra named parameters: strip0, err, spin_limit.
// ---------------------------------------------------------------------------------
#ifndef ST2B_SLOTS
#define ST2B_SLOTS 8
#endif
#ifndef ST2B_ROWS
#define ST2B_ROWS 64
#endif
extern __shared__ __align__(128) unsigned char st2b_smem[];
__device__ __forceinline__ u32 st2b_addr(const void* ptr) { return (u32)__cvta_generic_to_shared(ptr); }
__device__ __forceinline__ bool st2b_try_wait(u64* bar, u32 parity) {
  u32 ok;
  asm volatile(
      "{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(ok)
      : "r"(st2b_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void acc_bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(st2b_addr(dst)), "l"(src),
               "r"(bytes), "r"(st2b_addr(bar))
               : "memory");
}

// input row number I of the task (row y0 - ST_RYMAX + I of the arrays) goes to slot I % ST2B_SLOTS
#define ST2B_ISSUE(I)                                                                                  \
  {                                                                                                    \
    u64* bar_ = &bar[(I) % ST2B_SLOTS];                                                                \
    unsigned char* base_ = ring + (size_t)((I) % ST2B_SLOTS) * ST2_STAGE_BYTES;                        \
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(st2b_addr(bar_)), "r"((u32)ST2_STAGE_BYTES) : "memory"); \
    ST2_BULK_ISSUE_ALL(base_, bar_, y0 - ST_RYMAX + (I), gxw)                                          \
  }

#define ST2B_STEP(PH)                                                                                  \
  if ((PH) < ST_HW && i0 + (PH) < nrows && !failed) {                                                  \
    const int i = i0 + (PH);                                                                           \
    const int s = i % ST2B_SLOTS;                                                                      \
    const u32 par = (u32)(i / ST2B_SLOTS) & 1u;                                                        \
    i64 spins = 0;                                                                                     \
    while (!st2b_try_wait(&bar[s], par))                                                               \
      if (++spins > p.spin_limit) { failed = 1; break; }                                               \
    failed = __any_sync(ACC_FULL_MASK, failed);                                                        \
    if (!failed) {                                                                                     \
      done = i + 1;                                                                                    \
      ST2_TAKE_ALL((PH) % ST_HW, ring + (size_t)s * ST2_STAGE_BYTES, y0 - ST_RYMAX + i)                \
      ST2_COMMIT_ALL((PH) % ST_HW)   /* the shuffles use what was read: the slot is free */            \
      __syncwarp();                                                                                    \
      if (lane == 0 && i + ST2B_SLOTS < nrows) ST2B_ISSUE(i + ST2B_SLOTS)                              \
      if (i >= 2 * ST_RYMAX) {                                                                         \
        const int yy = y0 + i - 2 * ST_RYMAX;                                                          \
        elt_t o[4];                                                                                    \
        o[0] = ST2_apply<0, ((PH) + 2 * ST_HW - 2 * ST_RYMAX) % ST_HW>(p, ST2_WIN_ARGS);               \
        o[1] = ST2_apply<1, ((PH) + 2 * ST_HW - 2 * ST_RYMAX) % ST_HW>(p, ST2_WIN_ARGS);               \
        o[2] = ST2_apply<2, ((PH) + 2 * ST_HW - 2 * ST_RYMAX) % ST_HW>(p, ST2_WIN_ARGS);               \
        o[3] = ST2_apply<3, ((PH) + 2 * ST_HW - 2 * ST_RYMAX) % ST_HW>(p, ST2_WIN_ARGS);               \
        if (writer) OUT0_store4(p, (i64)yy * (i64)o2 + (i64)gx0, o);                                   \
      }                                                                                                \
    }                                                                                                  \
  }

extern "C" __global__ void __launch_bounds__(ST2_THREADS, ST2_MIN_BLOCKS) acc_stencil2d_bulk(const Params p) {
  __shared__ __align__(8) u64 bars[ST2_WARPS][ST2B_SLOTS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 task = (i64)blockIdx.x * ST2_WARPS + warp;
  if (task >= p.tiles1 * p.tiles2) return;
  const int o2 = (int)p.o2;
  const int rb = (int)(task / p.tiles2);
  const int strip = (int)p.strip0 + (int)(task - (i64)rb * p.tiles2);
  const int gxw = strip * ST2_STRIP - 4;              // first of the warp's 128 columns
  const int gx0 = gxw + lane * 4;
  const int y0 = (int)p.row0 + rb * ST2B_ROWS;
  const int y1 = min(y0 + ST2B_ROWS, (int)p.row1);
  const bool writer = lane >= 1 && lane <= 30;
  unsigned char* ring = st2b_smem + (size_t)warp * ((size_t)ST2B_SLOTS * ST2_STAGE_BYTES);
  u64* bar = bars[warp];
  if (lane == 0) {
    for (int s = 0; s < ST2B_SLOTS; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(st2b_addr(&bar[s])), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int nrows = (y1 - y0) + 2 * ST_RYMAX;         // input rows the task reads
  if (lane == 0)
    for (int i = 0; i < ST2B_SLOTS && i < nrows; ++i) ST2B_ISSUE(i)
  ST2_WIN_DECL
  int failed = 0;
  int done = 0;                                       // rows taken so far (every one of them had arrived)
  for (int i0 = 0; i0 < nrows && !failed; i0 += ST_HW) {
    ST2B_STEP(0) ST2B_STEP(1) ST2B_STEP(2) ST2B_STEP(3) ST2B_STEP(4) ST2B_STEP(5) ST2B_STEP(6) ST2B_STEP(7) ST2B_STEP(8)
  }
  if (failed) {
    // A copy did not arrive within the bound.  Report it, then give the copies still in flight into this
    // warp's slots a (much longer, still bounded) time to land before the shared memory is given up.
    if (lane == 0) {
      acc_fail(p.err, 110 /* ETIMEDOUT */);
      const int issued = min(nrows, done + ST2B_SLOTS);
      for (int i = done; i < issued; ++i) {
        i64 spins = 0;
        while (!st2b_try_wait(&bar[i % ST2B_SLOTS], (u32)(i / ST2B_SLOTS) & 1u))
          if (++spins > ((i64)1 << 26)) break;
      }
    }
    __syncwarp();
  }
}
#endif
