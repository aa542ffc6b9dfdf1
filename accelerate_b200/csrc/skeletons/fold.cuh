// fold / fold1 along the innermost dimension (Interpreter.hs:371-387).
//
// The combination function is only required to be associative, so every
// reduction below keeps operands in index order unless the generator proved
// the function commutative (ACC_COMMUTATIVE), in which case each lane keeps a
// private accumulator over interleaved positions.  A seed is applied exactly
// once per output element (it need not be neutral).
//
// Kernels:
//   acc_fold_all   one output element reduced by the whole grid; per-CTA
//                  partials in scratch, the last CTA to finish combines them
//                  in CTA order (a ticket counter, reset for the next launch).
//   acc_fold_rows  FOLD_G lanes per output element (FOLD_G = 1..32).
// HBM traffic: the stream bytes of one input element per element folded.

#define FOLD_THREADS 256
#define FOLD_WARPS (FOLD_THREADS / 32)
#define FOLD_TILE (FOLD_THREADS * 4)

__device__ __forceinline__ void fold_push(const Params& p, elt_t& v, bool& have, const elt_t& x) {
  if (have) v = F_combine(p, v, x);
  else { v = x; have = true; }
}
__device__ __forceinline__ void fold_merge(const Params& p, elt_t& v, bool& have, const elt_t& o, bool ohave) {
  if (ohave) fold_push(p, v, have, o);
}
// lanes [0, width) of each aligned group: lane 0 of the group receives v0 . v1 . ... in lane order
template <int WIDTH>
__device__ __forceinline__ void fold_group_reduce(const Params& p, elt_t& v, bool& have, int lane_in_group) {
#pragma unroll
  for (int d = 1; d < WIDTH; d <<= 1) {
    const elt_t o = acc_shfl_down(v, d);
    const int oh = __shfl_down_sync(ACC_FULL_MASK, (int)have, d);
    if (lane_in_group + d < WIDTH) fold_merge(p, v, have, o, oh != 0);
  }
}
// read a struct another CTA wrote (after the writer's fence and our ticket)
template <class T> __device__ __forceinline__ T fold_ld_shared_result(const T* src) {
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

// Reduce the values held by all threads of the CTA in thread order; the result
// is valid in thread 0.
__device__ __forceinline__ void fold_block_reduce(const Params& p, elt_t& v, bool& have, elt_t* sm_v, int* sm_h) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#if defined(FOLD_REDUX)
  {
    // 32-bit integer (+), min, max, and, or, xor: the warp's values combine in one redux.sync; lanes that hold
    // nothing contribute the operation's identity
    const unsigned holders = __ballot_sync(ACC_FULL_MASK, have);
    u32 x = FOLD_REDUX_IDENTITY, r;
    if (have) memcpy(&x, &v.l0, 4);
    asm volatile(FOLD_REDUX : "=r"(r) : "r"(x));
    memcpy(&v.l0, &r, 4);
    have = holders != 0;
  }
#else
  fold_group_reduce<32>(p, v, have, lane);
#endif
  if (lane == 0) { sm_v[warp] = v; sm_h[warp] = have; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < FOLD_WARPS; ++w) fold_merge(p, v, have, sm_v[w], sm_h[w] != 0);
  }
  __syncthreads();
}

// Reduce elements [e0, e1) of row `row` over the CTA; result valid in thread 0.
__device__ __forceinline__ void fold_span(const Params& p, i64 row, i64 e0, i64 e1, bool vec, elt_t& acc, bool& have,
                                          elt_t* sm_v, int* sm_h) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  have = false;
#if ACC_COMMUTATIVE
  i64 t = e0;
  if (vec) {
    // four tiles in flight per thread
    for (; t + 4 * FOLD_TILE <= e1; t += 4 * FOLD_TILE) {
      elt_t x[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) D0_get4(p, row, t + u * FOLD_TILE + tid * 4, x[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int k = 0; k < 4; ++k) fold_push(p, acc, have, x[u][k]);
      }
    }
    for (; t + FOLD_TILE <= e1; t += FOLD_TILE) {
      elt_t x[4];
      D0_get4(p, row, t + tid * 4, x);
#pragma unroll
      for (int k = 0; k < 4; ++k) fold_push(p, acc, have, x[k]);
    }
  }
  for (i64 j = t + tid; j < e1; j += FOLD_THREADS) fold_push(p, acc, have, D0_get(p, row, j));
  (void)lane; (void)warp;
#else
  // index order is kept: each warp owns a contiguous part of the span and walks it
  // in steps of 128 elements; lane 0 carries the running value.
  const i64 span = e1 - e0;
  const i64 per_warp = ((span + FOLD_WARPS * 128 - 1) / (FOLD_WARPS * 128)) * 128;
  const i64 w0 = e0 + warp * per_warp;
  i64 w1 = w0 + per_warp;
  if (w1 > e1) w1 = e1;
  for (i64 s = w0; s < w1; s += 128) {
    elt_t v;
    bool hv = false;
    const i64 j = s + lane * 4;
    if (vec && j + 4 <= w1) {
      elt_t x[4];
      D0_get4(p, row, j, x);
#pragma unroll
      for (int k = 0; k < 4; ++k) fold_push(p, v, hv, x[k]);
    } else {
      for (int k = 0; k < 4; ++k)
        if (j + k < w1) fold_push(p, v, hv, D0_get(p, row, j + k));
    }
    fold_group_reduce<32>(p, v, hv, lane);
    if (lane == 0) fold_merge(p, acc, have, v, hv);
  }
  // only lane 0 of each warp holds a value
  if (lane != 0) have = false;
#endif
  fold_block_reduce(p, acc, have, sm_v, sm_h);
}

// Named parameters: n (innermost extent), row (output element), vec,
// scratch (elt_t[gridDim.x]), flags (int[gridDim.x]), counter (u32*).
extern "C" __global__ void __launch_bounds__(FOLD_THREADS) acc_fold_all(const Params p) {
  __shared__ elt_t sm_v[FOLD_WARPS];
  __shared__ int sm_h[FOLD_WARPS];
  __shared__ int sm_last;
  const i64 n = p.n;
  const i64 ntiles = (n + FOLD_TILE - 1) / FOLD_TILE;
  const i64 per = (ntiles + gridDim.x - 1) / gridDim.x;
  i64 e0 = (i64)blockIdx.x * per * FOLD_TILE;
  i64 e1 = e0 + per * FOLD_TILE;
  if (e0 > n) e0 = n;
  if (e1 > n) e1 = n;
  elt_t acc;
  bool have;
  fold_span(p, p.row, e0, e1, p.vec != 0, acc, have, sm_v, sm_h);
  elt_t* partial = reinterpret_cast<elt_t*>(p.scratch);
  int* flags = reinterpret_cast<int*>(p.flags);
  unsigned* counter = reinterpret_cast<unsigned*>(p.counter);
  if (threadIdx.x == 0) {
    if (have) partial[blockIdx.x] = acc;
    flags[blockIdx.x] = have ? 1 : 0;
    __threadfence();
    const unsigned ticket = atomicAdd(counter, 1u);
    sm_last = (ticket == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  // the last CTA combines the partials in CTA order
  const int per_thread = ((int)gridDim.x + FOLD_THREADS - 1) / FOLD_THREADS;
  have = false;
  for (int c = threadIdx.x * per_thread; c < (threadIdx.x + 1) * per_thread && c < (int)gridDim.x; ++c) {
    const int h = *reinterpret_cast<const volatile int*>(flags + c);
    if (h) fold_push(p, acc, have, fold_ld_shared_result(partial + c));
  }
  fold_block_reduce(p, acc, have, sm_v, sm_h);
  if (threadIdx.x == 0) {
#if ACC_SEEDED
    const elt_t z = F_seed(p);
    OUT0_store(p, p.row, have ? F_combine(p, z, acc) : z);
#else
    if (have) OUT0_store(p, p.row, acc);
#endif
    *counter = 0u;
  }
}

#ifndef FOLD_G
#define FOLD_G 32
#endif
// Named parameters: n (innermost extent), rows (output elements), vec.
extern "C" __global__ void __launch_bounds__(FOLD_THREADS) acc_fold_rows(const Params p) {
  const i64 n = p.n, rows = p.rows;
  const bool vec = p.vec != 0;
  const int lane = threadIdx.x & 31;
  const int gl = lane % FOLD_G;           // lane within its group
  const int gw = lane / FOLD_G;           // group within the warp
  const int groups_per_warp = 32 / FOLD_G;
  const i64 warp_id = ((i64)blockIdx.x * FOLD_THREADS + threadIdx.x) >> 5;
  const i64 nwarps = ((i64)gridDim.x * FOLD_THREADS) >> 5;
  for (i64 r0 = warp_id * groups_per_warp; r0 < rows; r0 += nwarps * groups_per_warp) {
    const i64 row = r0 + gw;
    const bool active = row < rows;
    elt_t acc;
    bool have = false;
#if ACC_COMMUTATIVE
    if (active) {
      i64 j = 0;
      if (vec) {
        const i64 nvec = n & ~(i64)3;
        i64 jj = (i64)gl * 4;
        for (; jj + 3 * FOLD_G * 4 < nvec; jj += 4 * FOLD_G * 4) {
          elt_t x[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) D0_get4(p, row, jj + u * FOLD_G * 4, x[u]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int k = 0; k < 4; ++k) fold_push(p, acc, have, x[u][k]);
          }
        }
        for (; jj < nvec; jj += FOLD_G * 4) {
          elt_t x[4];
          D0_get4(p, row, jj, x);
#pragma unroll
          for (int k = 0; k < 4; ++k) fold_push(p, acc, have, x[k]);
        }
        j = nvec;
      }
      for (i64 q = j + gl; q < n; q += FOLD_G) fold_push(p, acc, have, D0_get(p, row, q));
    }
    fold_group_reduce<FOLD_G>(p, acc, have, gl);
#else
    // index order: the group walks the row in steps of FOLD_G * 4 elements
    const i64 steps = (n + FOLD_G * 4 - 1) / (FOLD_G * 4);
    i64 max_steps = steps;  // identical for every group of the warp (same n)
    for (i64 s = 0; s < max_steps; ++s) {
      elt_t v;
      bool hv = false;
      const i64 j = s * FOLD_G * 4 + (i64)gl * 4;
      if (active) {
        if (vec && j + 4 <= n) {
          elt_t x[4];
          D0_get4(p, row, j, x);
#pragma unroll
          for (int k = 0; k < 4; ++k) fold_push(p, v, hv, x[k]);
        } else {
          for (int k = 0; k < 4; ++k)
            if (j + k < n) fold_push(p, v, hv, D0_get(p, row, j + k));
        }
      }
      fold_group_reduce<FOLD_G>(p, v, hv, gl);
      if (gl == 0) fold_merge(p, acc, have, v, hv);
    }
#endif
    if (active && gl == 0) {
#if ACC_SEEDED
      const elt_t z = F_seed(p);
      OUT0_store(p, row, have ? F_combine(p, z, acc) : z);
#else
      if (have) OUT0_store(p, row, acc);
#endif
    }
  }
}
