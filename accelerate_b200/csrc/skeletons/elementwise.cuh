// generate / map / zipWith / backpermute / transform: one elementwise skeleton.
// Follows fromFunctionM (Representation/Array.hs:109-122): out[i] = f (fromIndex sh i).
//
// Named parameters: n (elements), vec (1: every stream has the output's shape
// and the innermost extent is a multiple of 4, so four consecutive outputs are
// four consecutive, 16-byte aligned addresses of every stream).
// HBM traffic: sum of stream element sizes + output element size per element.

#define GEN_THREADS 256

extern "C" __global__ void __launch_bounds__(GEN_THREADS) acc_generate(const Params p) {
  const i64 n = p.n;
  const i64 inner = D0_INNER;
  const i64 tid = (i64)blockIdx.x * GEN_THREADS + threadIdx.x;
  const i64 nthreads = (i64)gridDim.x * GEN_THREADS;
  i64 done = 0;
  if (p.vec) {
    const i64 nv = n >> 2;
    for (i64 v = tid; v < nv; v += nthreads) {
      const i64 i = v << 2;
      i64 row = 0, j = i;
      if (inner != n) { row = i / inner; j = i - row * inner; }
      elt_t o[4];
      D0_get4(p, row, j, o);
      OUT0_store4(p, i, o);
    }
    done = nv << 2;
  }
  for (i64 i = done + tid; i < n; i += nthreads) {
    i64 row = 0, j = i;
    if (inner != n) { row = i / inner; j = i - row * inner; }
    OUT0_store(p, i, D0_get(p, row, j));
  }
}
