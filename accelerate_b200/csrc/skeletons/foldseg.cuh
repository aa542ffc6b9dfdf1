// foldSeg / fold1Seg (Interpreter.hs:390-424).  The descriptor operand D1 holds
// segment OFFSETS (length = segments + 1); segment j of every outer slice covers
// inner positions [off[j], off[j+1]).  FOLDSEG_G lanes cooperate on one segment.
//
// Commutative functions: unaligned head, 128-bit aligned body, tail; lanes keep
// private accumulators.  Otherwise the group walks the segment in index order.
// Named parameters: segs, rows, vec, err.
// HBM traffic: input stream bytes per element + 2 offsets per segment.

#define FSEG_THREADS 256
#ifndef FOLDSEG_G
#define FOLDSEG_G 32
#endif
#define ACC_ERR_EMPTY_SEGMENT 1001

__device__ __forceinline__ void fseg_push(const Params& p, elt_t& v, bool& have, const elt_t& x) {
  if (have) v = F_combine(p, v, x);
  else { v = x; have = true; }
}
__device__ __forceinline__ void fseg_group_reduce(const Params& p, elt_t& v, bool& have, int gl) {
#pragma unroll
  for (int d = 1; d < FOLDSEG_G; d <<= 1) {
    const elt_t o = acc_shfl_down(v, d);
    const int oh = __shfl_down_sync(ACC_FULL_MASK, (int)have, d);
    if (gl + d < FOLDSEG_G && oh) fseg_push(p, v, have, o);
  }
}

extern "C" __global__ void __launch_bounds__(FSEG_THREADS) acc_foldseg(const Params p) {
  const i64 segs = p.segs, total = p.rows * segs;
  const bool vec = p.vec != 0;
  const int lane = threadIdx.x & 31;
  const int gl = lane % FOLDSEG_G, gw = lane / FOLDSEG_G;
  const int gpw = 32 / FOLDSEG_G;
  const i64 warp_id = ((i64)blockIdx.x * FSEG_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * FSEG_THREADS) >> 5;
  for (i64 s0 = warp_id * gpw; s0 < total; s0 += nwarps * gpw) {
    const i64 s = s0 + gw;
    const bool active = s < total;
    i64 row = 0, seg = 0, start = 0, end = 0;
    if (active) {
      row = s / segs;
      seg = s - row * segs;
      start = (i64)D1_get(p, 0, seg).l0;
      end = (i64)D1_get(p, 0, seg + 1).l0;
    }
    elt_t acc;
    bool have = false;
#if ACC_COMMUTATIVE
    if (active) {
      i64 j0 = vec ? ((start + 3) & ~(i64)3) : end;
      if (j0 > end) j0 = end;
      for (i64 j = start + gl; j < j0; j += FOLDSEG_G) fseg_push(p, acc, have, D0_get(p, row, j));
      i64 jj = j0 + (i64)gl * 4;
      for (; jj + 3 * FOLDSEG_G * 4 + 4 <= end; jj += 4 * FOLDSEG_G * 4) {
        elt_t x[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) D0_get4(p, row, jj + u * FOLDSEG_G * 4, x[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int k = 0; k < 4; ++k) fseg_push(p, acc, have, x[u][k]);
        }
      }
      for (; jj + 4 <= end; jj += FOLDSEG_G * 4) {
        elt_t x[4];
        D0_get4(p, row, jj, x);
#pragma unroll
        for (int k = 0; k < 4; ++k) fseg_push(p, acc, have, x[k]);
      }
      const i64 j1 = j0 + ((end - j0) & ~(i64)3);
      for (i64 j = j1 + gl; j < end; j += FOLDSEG_G) fseg_push(p, acc, have, D0_get(p, row, j));
    }
    fseg_group_reduce(p, acc, have, gl);
#else
    // steps must be uniform across the warp: use the longest segment among its groups
    i64 len = active ? end - start : 0;
    if (len < 0) len = 0;
    i64 maxlen = len;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const i64 o = __shfl_xor_sync(ACC_FULL_MASK, maxlen, d);
      if (o > maxlen) maxlen = o;
    }
    for (i64 t = 0; t < maxlen; t += FOLDSEG_G) {
      elt_t v;
      bool hv = false;
      const i64 j = start + t + gl;
      if (active && j < end) { v = D0_get(p, row, j); hv = true; }
      fseg_group_reduce(p, v, hv, gl);
      if (gl == 0 && hv) fseg_push(p, acc, have, v);
    }
#endif
    if (active && gl == 0) {
#if ACC_SEEDED
      const elt_t z = F_seed(p);
      OUT0_store(p, s, have ? F_combine(p, z, acc) : z);
#else
      if (have) OUT0_store(p, s, acc);
      else acc_fail(p.err, ACC_ERR_EMPTY_SEGMENT);   // "empty segment", Interpreter.hs:423
#endif
    }
  }
}
