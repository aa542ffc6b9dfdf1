// permute (Interpreter.hs:585-624): the output starts as a copy of the defaults
// (made by the host before this kernel); every source element whose index
// function yields `Just ix` is combined into out[ix] as `f new old`.
//
// How the update is applied (PERMUTE_MODE, chosen by the code generator):
//   PERMUTE_ATOMIC_*  f is (+)/min/max/and/or/xor on a 32/64-bit scalar: one
//                     fire-and-forget reduction (red.global), optionally staged
//                     through a CTA-private copy of the first `priv` target
//                     elements in shared memory when the target is small
//                     (PERMUTE_SMEM); for (+) on 32-bit integers a private copy of
//                     16-bit fields covers targets twice that size (PERMUTE_SMEM16);
//   PERMUTE_CAS       any other f on a 32/64-bit scalar: compare-and-swap loop;
//   PERMUTE_STORE     `permute const`: plain store (targets assumed unique);
//   PERMUTE_LOCK      everything else (tuples, narrow types): one spin lock per
//                     target element, bounded by `spin_limit`.
// f must be associative and commutative (Language.hs:707), so update order is free.
//
// Named parameters: n, vec, out_n, priv, locks, err, spin_limit.
// HBM traffic: source stream bytes per element (+ the target, amortised).

#ifndef PERMUTE_THREADS
#define PERMUTE_THREADS 512
#endif
#define PERMUTE_ATOMIC_ADD 1
#define PERMUTE_ATOMIC_MIN 2
#define PERMUTE_ATOMIC_MAX 3
#define PERMUTE_ATOMIC_AND 4
#define PERMUTE_ATOMIC_OR 5
#define PERMUTE_ATOMIC_XOR 6
#define PERMUTE_CAS 7
#define PERMUTE_STORE 8
#define PERMUTE_LOCK 9
#ifndef PERMUTE_SMEM
#define PERMUTE_SMEM 0
#endif
#ifndef PERMUTE_UNROLL
#define PERMUTE_UNROLL 4
#endif
#define PERMUTE_IS_ATOMIC (PERMUTE_MODE >= PERMUTE_ATOMIC_ADD && PERMUTE_MODE <= PERMUTE_ATOMIC_XOR)

#if PERMUTE_IS_ATOMIC || PERMUTE_MODE == PERMUTE_CAS
#if PERMUTE_BYTES == 4
typedef u32 permute_word;
#else
typedef u64 permute_word;
#endif
__device__ __forceinline__ permute_word permute_bits(PERMUTE_T v) { return *reinterpret_cast<permute_word*>(&v); }
__device__ __forceinline__ PERMUTE_T permute_val(permute_word w) { return *reinterpret_cast<PERMUTE_T*>(&w); }
#endif

#if PERMUTE_IS_ATOMIC
// works on global and shared addresses alike
__device__ __forceinline__ void permute_atomic(PERMUTE_T* addr, PERMUTE_T v) {
#if PERMUTE_MODE == PERMUTE_ATOMIC_ADD
#if PERMUTE_FLOAT
  atomicAdd(addr, v);
#else
  atomicAdd(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#endif
#elif PERMUTE_MODE == PERMUTE_ATOMIC_MIN
#if PERMUTE_SIGNED && PERMUTE_BYTES == 4
  atomicMin(reinterpret_cast<int*>(addr), (int)v);
#elif PERMUTE_SIGNED
  atomicMin(reinterpret_cast<long long*>(addr), (long long)v);
#else
  atomicMin(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#endif
#elif PERMUTE_MODE == PERMUTE_ATOMIC_MAX
#if PERMUTE_SIGNED && PERMUTE_BYTES == 4
  atomicMax(reinterpret_cast<int*>(addr), (int)v);
#elif PERMUTE_SIGNED
  atomicMax(reinterpret_cast<long long*>(addr), (long long)v);
#else
  atomicMax(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#endif
#elif PERMUTE_MODE == PERMUTE_ATOMIC_AND
  atomicAnd(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#elif PERMUTE_MODE == PERMUTE_ATOMIC_OR
  atomicOr(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#else
  atomicXor(reinterpret_cast<permute_word*>(addr), permute_bits(v));
#endif
}
// the value that leaves a target element unchanged
__device__ __forceinline__ PERMUTE_T permute_identity() {
#if PERMUTE_MODE == PERMUTE_ATOMIC_MIN
#if PERMUTE_SIGNED
  return (PERMUTE_T)(((permute_word)1 << (PERMUTE_BYTES * 8 - 1)) - 1);
#else
  return (PERMUTE_T)~(permute_word)0;
#endif
#elif PERMUTE_MODE == PERMUTE_ATOMIC_MAX
#if PERMUTE_SIGNED
  return permute_val((permute_word)1 << (PERMUTE_BYTES * 8 - 1));
#else
  return (PERMUTE_T)0;
#endif
#elif PERMUTE_MODE == PERMUTE_ATOMIC_AND
  return permute_val(~(permute_word)0);
#else
  return (PERMUTE_T)0;
#endif
}
#endif

#ifndef PERMUTE_SMEM16
#define PERMUTE_SMEM16 0
#endif
#if PERMUTE_SMEM || PERMUTE_SMEM16
extern __shared__ __align__(16) unsigned char permute_smem_raw[];
#endif

#if PERMUTE_SMEM16
// (+) on a 32-bit integer target of up to twice as many elements as a CTA has shared-memory words.
// The CTA has a private copy of EVERY element, wherever the frequent ones lie: it keeps the LOW 16
// bits of its contribution, two elements per word, and sends everything else straight to the
// target with red.global:
//   * the high 16 bits of an addend (zero for counts and other small addends);
//   * 65536 whenever a 16-bit field wraps.  Every update is one atomicAdd on the word, whose return
//     value shows exactly whether the addressed field wrapped; a wrap of the lower field also
//     carries 1 into the upper field, which is taken out again with a second atomic (and if that
//     carry or its removal wraps the upper field, that too is seen in the returned value and
//     compensated).  All arithmetic is modulo 2^32 on the target, like the reference's Int32/Word32.
// At the end the fields are added to the target.
// The update is split in two so that a thread can have the atomics of all its elements in flight
// before it looks at any of their results: permute_issue16 performs the atomic and hands back the
// word it found, permute_settle16 does what that word demands.
__device__ __forceinline__ u32* permute_fields16(const Params& p) { (void)p; return reinterpret_cast<u32*>(permute_smem_raw); }
__device__ __forceinline__ u32 permute_issue16(const Params& p, i64 dst, u32 v) {
  const i64 f = dst;
  const u32 lo = v & 0xffffu;
  return atomicAdd(permute_fields16(p) + (f >> 1), (f & 1) ? (lo << 16) : lo);
}
__device__ __forceinline__ void permute_settle16(const Params& p, i64 dst, u32 v, u32 old) {
  const i64 f = dst;
  u32* out = reinterpret_cast<u32*>(p.out0_l0);
  const u32 hi = v & 0xffff0000u, lo = v & 0xffffu;
  if (hi) atomicAdd(out + dst, hi);
  if (f & 1) {
    if (((old >> 16) + lo) >> 16) atomicAdd(out + dst, 65536u);
  } else if (((old & 0xffffu) + lo) >> 16) {
    atomicAdd(out + dst, 65536u);
    if ((old >> 16) == 0xffffu) atomicAdd(out + dst + 1, 65536u);        // the carry wrapped the upper field
    const u32 old2 = atomicAdd(permute_fields16(p) + (f >> 1), 0xffff0000u);   // take the carry out again
    if ((old2 >> 16) == 0u) atomicAdd(out + dst + 1, 0u - 65536u);       // ... which wrapped it downwards
  }
}
__device__ __forceinline__ void permute_add16(const Params& p, i64 dst, u32 v) {
  permute_settle16(p, dst, v, permute_issue16(p, dst, v));
}
#endif


__device__ __forceinline__ void permute_update(const Params& p, i64 dst, const elt_t& v) {
#if PERMUTE_IS_ATOMIC
#if PERMUTE_SMEM16
  permute_add16(p, dst, permute_bits(v.l0));
  return;
#endif
#if PERMUTE_SMEM
  if (dst < p.priv) { permute_atomic(reinterpret_cast<PERMUTE_T*>(permute_smem_raw) + dst, v.l0); return; }
#endif
  permute_atomic(p.out0_l0 + dst, v.l0);
#elif PERMUTE_MODE == PERMUTE_CAS
  permute_word* a = reinterpret_cast<permute_word*>(p.out0_l0 + dst);
  permute_word old = *reinterpret_cast<volatile permute_word*>(a), assumed;
  do {
    assumed = old;
    elt_t cur;
    cur.l0 = permute_val(assumed);
    const elt_t nv = F_combine(p, v, cur);
    old = atomicCAS(a, assumed, permute_bits(nv.l0));
  } while (assumed != old);
#elif PERMUTE_MODE == PERMUTE_STORE
  OUT0_store(p, dst, v);
#else
  unsigned* lock = reinterpret_cast<unsigned*>(p.locks) + dst;
  i64 spins = 0;
  for (;;) {
    if (atomicCAS(lock, 0u, 1u) == 0u) {
      __threadfence();
      const elt_t cur = OUT0_load(p, dst);
      OUT0_store(p, dst, F_combine(p, v, cur));
      __threadfence();
      atomicExch(lock, 0u);
      break;
    }
    if (++spins > p.spin_limit) { acc_fail(p.err, 110 /* ETIMEDOUT */); break; }
    __nanosleep(40);
  }
#endif
}

__device__ __forceinline__ void permute_elem(const Params& p, const pelem_t& e, bool& outside) {
  // the reference checks every component of the target index (indexCheck in toIndex,
  // Shape.hs:102-106); the generated index function yields -1 for a target outside the array.
  // The thread only notes the fact here and reports it once, after its loop.
  if (e.l0 != 0) {
    if ((u64)e.l1 < (u64)p.out_n) permute_update(p, e.l1, P_value(e));
    else outside = true;
  }
}

// Which of two kernels handles a target that the 32-bit private copy covers only in part?  The copy
// of the first `priv` elements is the faster one as long as almost every update lands inside it;
// updates outside go to the target one by one, and a frequent element out there serialises them.
// The copy of 16-bit fields covers everything but pays for updates whose result it must inspect.
// acc_permute_sample looks at 65 536 source elements spread over the input and writes 1 to
// *choice if more than 1 in 64 of their targets lie outside the first `priv` elements, else 0; both
// kernels are launched behind it and the one that is not chosen returns at once (no host round trip).
#if defined(PERMUTE_SAMPLE) && PERMUTE_SAMPLE
// One sample per thread, ceil(samples / 1024) CTAs (a single CTA walking all 65 536 samples took 90 us:
// every sample is a separate sector).  `choice` points at three words: the verdict, the count so far and a
// ticket; the CTA that draws the last ticket writes the verdict and clears the other two for the next launch.
extern "C" __global__ void __launch_bounds__(1024) acc_permute_sample(const Params p) {
  __shared__ u32 outside;
  const i64 n = p.n, inner = P_INNER;
  if (threadIdx.x == 0) outside = 0u;
  __syncthreads();
  const i64 samples = n < 65536 ? n : 65536;
  const i64 step = n / samples;
  const i64 k = (i64)blockIdx.x * 1024 + threadIdx.x;
  bool out = false;
  if (k < samples) {
    // one element from every stretch of `step`, at a position that depends on k: a regular stride can fall
    // into step with a period of the data and then sees the same few elements over and over
    const i64 i = k * step + (i64)((((u64)k * 0x9E3779B97F4A7C15ull) >> 33) % (u64)step);
    i64 row = 0, j = i;
    if (inner != n) { row = i / inner; j = i - row * inner; }
    const pelem_t e = P_get(p, row, j);
    out = e.l0 != 0 && e.l1 >= p.priv;
  }
  const unsigned m = __ballot_sync(ACC_FULL_MASK, out);
  if ((threadIdx.x & 31) == 0 && m) atomicAdd(&outside, (u32)__popc(m));
  __syncthreads();
  if (threadIdx.x == 0) {
    int* w = reinterpret_cast<int*>(p.choice);
    if (outside) atomicAdd(&w[1], (int)outside);
    __threadfence();
    if (atomicAdd(&w[2], 1) == (int)gridDim.x - 1) {
      __threadfence();
      const i64 total = atomicExch(&w[1], 0);
      w[0] = total * 64 > samples ? 1 : 0;
      w[2] = 0;
    }
  }
}
#endif
#ifndef PERMUTE_CHOICE_ID
#define PERMUTE_CHOICE_ID 0
#endif

extern "C" __global__ void __launch_bounds__(PERMUTE_THREADS) acc_permute(const Params p) {
  if (p.choice != 0 && *reinterpret_cast<const volatile int*>(p.choice) != PERMUTE_CHOICE_ID) return;
  const i64 n = p.n;
  const i64 inner = P_INNER;
  const i64 tid = (i64)blockIdx.x * PERMUTE_THREADS + threadIdx.x;
  const i64 nthreads = (i64)gridDim.x * PERMUTE_THREADS;
#if PERMUTE_SMEM16
  {
    // p.priv16 words of two 16-bit fields each
    u32* sm16 = reinterpret_cast<u32*>(permute_smem_raw);
    for (i64 b = threadIdx.x; b < p.priv16; b += PERMUTE_THREADS) sm16[b] = 0u;
    __syncthreads();
  }
#endif
#if PERMUTE_SMEM
  PERMUTE_T* sm = reinterpret_cast<PERMUTE_T*>(permute_smem_raw);
  for (i64 b = threadIdx.x; b < p.priv; b += PERMUTE_THREADS) sm[b] = permute_identity();
  __syncthreads();
#endif
  i64 done = 0;
  bool outside = false;             // some target index of this thread lay outside the array
  if (p.vec) {
    const i64 nv = n >> 2;
    i64 v = tid;
    // PERMUTE_UNROLL 128-bit groups in flight per thread
    for (; v + (PERMUTE_UNROLL - 1) * nthreads < nv; v += PERMUTE_UNROLL * nthreads) {
      pelem_t x[PERMUTE_UNROLL][4];
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
        const i64 i = (v + u * nthreads) << 2;
        i64 row = 0, j = i;
        if (inner != n) { row = i / inner; j = i - row * inner; }
        P_get4(p, row, j, x[u]);
      }
#if PERMUTE_SMEM16
      u32 found[PERMUTE_UNROLL][4];
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const pelem_t& e = x[u][k];
          if (e.l0 != 0 && (u64)e.l1 < (u64)p.out_n) found[u][k] = permute_issue16(p, e.l1, permute_bits(P_value(e).l0));
        }
      }
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const pelem_t& e = x[u][k];
          if (e.l0 != 0) {
            if ((u64)e.l1 >= (u64)p.out_n) outside = true;
            else permute_settle16(p, e.l1, permute_bits(P_value(e).l0), found[u][k]);
          }
        }
      }
#else
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
#pragma unroll
        for (int k = 0; k < 4; ++k) permute_elem(p, x[u][k], outside);
      }
#endif
    }
    for (; v < nv; v += nthreads) {
      const i64 i = v << 2;
      i64 row = 0, j = i;
      if (inner != n) { row = i / inner; j = i - row * inner; }
      pelem_t x[4];
      P_get4(p, row, j, x);
#pragma unroll
      for (int k = 0; k < 4; ++k) permute_elem(p, x[k], outside);
    }
    done = nv << 2;
  }
  for (i64 i = done + tid; i < n; i += nthreads) {
    i64 row = 0, j = i;
    if (inner != n) { row = i / inner; j = i - row * inner; }
    permute_elem(p, P_get(p, row, j), outside);
  }
  if (outside) acc_fail(p.err, 1003 /* index out of bounds */);
#if PERMUTE_SMEM
  __syncthreads();
  for (i64 b = threadIdx.x; b < p.priv; b += PERMUTE_THREADS) {
    const PERMUTE_T v = sm[b];
    if (permute_bits(v) != permute_bits(permute_identity())) permute_atomic(p.out0_l0 + b, v);
  }
#endif
#if PERMUTE_SMEM16
  __syncthreads();
  {
    const u32* sm16 = permute_fields16(p);
    u32* out = reinterpret_cast<u32*>(p.out0_l0);
    for (i64 b = threadIdx.x; b < p.priv16; b += PERMUTE_THREADS) {
      const u32 w = sm16[b];
      const i64 dst = 2 * b;
      if (w & 0xffffu) atomicAdd(out + dst, w & 0xffffu);
      if ((w >> 16) && dst + 1 < p.out_n) atomicAdd(out + dst + 1, w >> 16);
    }
  }
#endif
}

