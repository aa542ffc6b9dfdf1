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
// output columns), vec (o2 % 4 == 0, 16-byte aligned output).
// One warp per task: grid = ceil(tiles1 * tiles2 / ST2_WARPS).

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
  const i64 ntasks = p.tiles1 * p.tiles2;
  const i64 task = (i64)blockIdx.x * ST2_WARPS + warp;
  if (task >= ntasks) return;
  const int o1 = (int)p.o1, o2 = (int)p.o2;
  const int rb = (int)(task / p.tiles2);
  const int strip = (int)(task - (i64)rb * p.tiles2);
  const int gx0 = strip * ST2_STRIP - 4 + lane * 4;
  const int y0 = (int)p.row0 + rb * ST2_ROWS;
  const int y1 = min(y0 + ST2_ROWS, (int)p.row1);
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
