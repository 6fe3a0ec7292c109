// Host-level array operations: the counterparts of cuTile.jl's `ct.Tiled` broadcast (src/broadcast.jl: a whole
// broadcast expression fused into one kernel) and mapreduce (src/mapreduce.jl: sum / prod / maximum / minimum / a
// mapped reduction over any set of dimensions).  The reference compiles the Julia expression; a prebuilt library
// cannot, so the expression arrives as a short postfix program (push input, push constant, unary function, binary
// operator).  The host turns it into instructions of an accumulator machine (compile_program below: a leaf operand
// of a binary operator is read in place, only a binary operator between two computed values touches the stack),
// and every thread runs those instructions on registers for four or eight elements at a time: still one pass over
// memory, one kernel, whatever the expression.  Arrays have up to three dimensions, column-major, first dimension
// contiguous; an operand with extent 1 along a dimension is expanded along it (stride 0).  Arithmetic is f32
// whatever the element type.  Both are bound by HBM bandwidth: bytes of the operands read once plus the result.
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>
#include <type_traits>

#include "ctx.h"

using namespace ctb_internal;

namespace {

constexpr int kMaxOps = CTB_TILED_MAX_OPS;
constexpr int kMaxInputs = CTB_TILED_MAX_INPUTS;
constexpr int kMaxConsts = CTB_TILED_MAX_CONSTS;
constexpr int kStack = 4;

// One instruction word of the accumulator machine.  The accumulator A is the top of a four-entry register stack.
//   kind LOAD : push; A = operand
//   kind UNARY: A = code(A)
//   kind BIN  : A = A code operand, or operand code A when the REV bit is set; an operand from the stack is popped
// operand source: the stack entry below A (BIN only), inputs[arg] or constants[arg].
enum : unsigned { K_LOAD = 0, K_UNARY = 1, K_BIN = 2 };
enum : unsigned { SRC_STACK = 0, SRC_INPUT = 1, SRC_CONST = 2 };
constexpr unsigned kRevBit = 1u << 4;
// Bits 24..31: the index the vector kernel switches on, dense so that the switch is one jump through a table:
// 0, 1 = push an input / a constant; 2..13 = the unary codes NEG..ABS2; then the seven binary codes for each of the six
// (operand source, reversed) pairs.
constexpr unsigned kDispatchUnary = 2, kDispatchBinary = 14;
__host__ __device__ constexpr unsigned bin_variant(unsigned src, bool rev) {
  return (src == SRC_INPUT ? 0u : src == SRC_CONST ? 1u : 2u) * 2u + (rev ? 1u : 0u);
}
__host__ __device__ constexpr unsigned dispatch_index(unsigned kind, unsigned src, bool rev, unsigned code) {
  return kind == K_LOAD ? (src == SRC_INPUT ? 0u : 1u)
         : kind == K_UNARY ? kDispatchUnary + (code - CTB_TILED_NEG)
                           : kDispatchBinary + 7u * bin_variant(src, rev) + (code - CTB_TILED_ADD);
}
__host__ __device__ constexpr unsigned make_ins(unsigned kind, unsigned src, bool rev, unsigned code, unsigned arg) {
  return kind | (src << 2) | (rev ? kRevBit : 0u) | (code << 8) | (arg << 16) | (dispatch_index(kind, src, rev, code) << 24);
}

struct Program {
  int n_ins;
  unsigned ins[kMaxOps];
  float consts[kMaxConsts];
};

struct Operands {
  const void* ptr[kMaxInputs];
  long long stride[kMaxInputs][3];
};

// ---- postfix program -> accumulator-machine instructions (host) ---------------------------------------------------
struct Node {
  int op, arg, left, right;  // left/right: node indices, -1 for none
  int need;                  // stack entries the subtree needs when it is evaluated into A
};
inline bool is_leaf(const Node& n) { return n.op == CTB_TILED_INPUT || n.op == CTB_TILED_CONST; }
inline unsigned leaf_src(const Node& n) { return n.op == CTB_TILED_INPUT ? SRC_INPUT : SRC_CONST; }

struct Compiler {
  Node nodes[kMaxOps];
  int n_nodes = 0;
  Program* out = nullptr;
  void put(unsigned w) { out->ins[out->n_ins++] = w; }
  void emit(int i) {
    const Node& n = nodes[i];
    if (is_leaf(n)) {
      put(make_ins(K_LOAD, leaf_src(n), false, 0, (unsigned)n.arg));
    } else if (n.right < 0) {
      emit(n.left);
      if (n.op != CTB_TILED_IDENTITY) put(make_ins(K_UNARY, 0, false, (unsigned)n.op, 0));
    } else {
      const Node &l = nodes[n.left], &r = nodes[n.right];
      const bool commutes = n.op == CTB_TILED_ADD || n.op == CTB_TILED_MUL;  // a op b == b op a bit for bit
      if (is_leaf(r)) {         // A = left; A = A op leaf
        emit(n.left);
        put(make_ins(K_BIN, leaf_src(r), false, (unsigned)n.op, (unsigned)r.arg));
      } else if (is_leaf(l)) {  // A = right; A = leaf op A
        emit(n.right);
        put(make_ins(K_BIN, leaf_src(l), !commutes, (unsigned)n.op, (unsigned)l.arg));
      } else if (l.need > r.need) {  // the deeper side first: A = right, below it left; A = below op A
        emit(n.left);
        emit(n.right);
        put(make_ins(K_BIN, SRC_STACK, !commutes, (unsigned)n.op, 0));
      } else {                  // A = left, below it right; A = A op below
        emit(n.right);
        emit(n.left);
        put(make_ins(K_BIN, SRC_STACK, false, (unsigned)n.op, 0));
      }
    }
  }
};

// Returns 0, or a negative number -(k+1) naming the offending postfix operation k with *why set; -1000 when the
// expression needs more than kStack live values.  *need: the stack entries the instructions use (1 = the accumulator
// alone).
int compile_program(const int32_t* program, int n_ops, int n_inputs, int n_constants, Program* out, const char** why,
                    int* need = nullptr) {
  Compiler c;
  c.out = out;
  out->n_ins = 0;
  int stack[kMaxOps], depth = 0;
  for (int k = 0; k < n_ops; ++k) {
    const int op = program[2 * k], arg = program[2 * k + 1];
    Node n = {op, arg, -1, -1, 1};
    if (op == CTB_TILED_INPUT) {
      if (arg < 0 || arg >= n_inputs) { *why = "names an input that was not given"; return -(k + 1); }
    } else if (op == CTB_TILED_CONST) {
      if (arg < 0 || arg >= n_constants) { *why = "names a constant that was not given"; return -(k + 1); }
    } else if (op >= CTB_TILED_IDENTITY && op <= CTB_TILED_ABS2) {
      if (depth < 1) { *why = "finds an empty stack"; return -(k + 1); }
      n.left = stack[--depth];
      n.need = c.nodes[n.left].need;
    } else if (op >= CTB_TILED_ADD && op <= CTB_TILED_POW) {
      if (depth < 2) { *why = "needs two values on the stack"; return -(k + 1); }
      n.right = stack[--depth];
      n.left = stack[--depth];
      const Node &l = c.nodes[n.left], &r = c.nodes[n.right];
      if (is_leaf(r)) n.need = l.need;
      else if (is_leaf(l)) n.need = r.need;
      else n.need = std::max(std::max(l.need, r.need), std::min(l.need, r.need) + 1);
    } else {
      *why = "is not an operation code";
      return -(k + 1);
    }
    c.nodes[c.n_nodes] = n;
    stack[depth++] = c.n_nodes++;
  }
  if (depth != 1) { *why = "the program must leave exactly one value"; return -(n_ops + 1); }
  if (c.nodes[stack[0]].need > kStack) return -1000;
  if (need) *need = c.nodes[stack[0]].need;
  c.emit(stack[0]);
  return 0;
}

__device__ __forceinline__ float unary(int op, float x) {
  switch (op) {
    case CTB_TILED_NEG: return -x;
    case CTB_TILED_ABS: return fabsf(x);
    case CTB_TILED_SQRT: return sqrtf(x);
    case CTB_TILED_EXP: return expf(x);
    case CTB_TILED_EXP2: return exp2f(x);
    case CTB_TILED_LOG: return logf(x);
    case CTB_TILED_LOG2: return log2f(x);
    case CTB_TILED_SIN: return sinf(x);
    case CTB_TILED_COS: return cosf(x);
    case CTB_TILED_TANH: return tanhf(x);
    case CTB_TILED_INV: return 1.0f / x;
    case CTB_TILED_ABS2: return x * x;
    default: return x;  // CTB_TILED_IDENTITY
  }
}
__device__ __forceinline__ float binary(int op, float a, float b) {
  switch (op) {
    case CTB_TILED_ADD: return a + b;
    case CTB_TILED_SUB: return a - b;
    case CTB_TILED_MUL: return a * b;
    case CTB_TILED_DIV: return a / b;
    case CTB_TILED_MAX: return fmaxf(a, b);
    case CTB_TILED_MIN: return fminf(a, b);
    default: return powf(a, b);  // CTB_TILED_POW
  }
}

template <typename T>
__device__ __forceinline__ float load1(const void* p, long long i) {
  if constexpr (sizeof(T) == 4) return static_cast<const float*>(p)[i];
  else return __half2float(static_cast<const __half*>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void store1(void* p, long long i, float v) {
  if constexpr (sizeof(T) == 4) static_cast<float*>(p)[i] = v;
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

// The general path, for arrays the vector path below cannot take (a first extent that is not a multiple of four, rows
// that do not start on 16-byte boundaries): instantiated with V = 1, G = 1, NIN = 4, DEEP = true, one element per
// thread and trip, operands and stack in registers.  (V = 4 groups of four neighbouring elements, G groups per thread
// and NIN operands held are the knobs of the register-only vector kernel this one was before the operands moved to
// shared memory; they still compile.)
// DENSE: every operand either has the destination's shape (dense) or is a single element: one linear index, no
// division.  Otherwise the group index is split into its three coordinates (32-bit arithmetic; the host checks
// that the element count fits).  The operands are read once per element into registers.
template <typename T, int V, int G, bool DENSE, int NIN, bool DEEP>
__global__ void __launch_bounds__(256)
    tiled_broadcast_kernel(void* __restrict__ dest, const Operands in, const Program prog, int n_inputs, long long d0,
                           long long d1, long long d2) {
  constexpr int E = V * G;
  constexpr int ES = DEEP ? E : 1;  // extent of the stack entries below the accumulator
  const long long n0 = d0 / V, total = n0 * d1 * d2;
  const long long grid_stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += grid_stride * G) {
    long long o[G];  // element offset of each group in the destination
    bool live[G];
    float x[NIN][E];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long ig = i + g * grid_stride;
      live[g] = ig < total;
      long long off[NIN];
      long long st0[NIN];
      if (DENSE) {
        o[g] = ig * V;
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
          st0[a] = in.stride[a][0];
          off[a] = st0[a] ? o[g] : 0;
        }
      } else {
        const unsigned u = (unsigned)ig, un0 = (unsigned)n0, ud1 = (unsigned)d1;
        const unsigned r = u / un0, i0 = (u - r * un0) * V, i2 = r / ud1, i1 = r - i2 * ud1;
        o[g] = i0 + d0 * (i1 + d1 * (long long)i2);
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
          st0[a] = in.stride[a][0];
          off[a] = i0 * st0[a] + i1 * in.stride[a][1] + i2 * in.stride[a][2];
        }
      }
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        float* xa = &x[a][g * V];
        if (a < n_inputs && live[g]) {
          if (V == 4 && st0[a] == 1) {
            if constexpr (sizeof(T) == 4) {
              const float4 q = __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(in.ptr[a]) + off[a]));
              xa[0] = q.x; xa[1 % V] = q.y; xa[2 % V] = q.z; xa[3 % V] = q.w;
            } else {
              const uint2 q = __ldcs(reinterpret_cast<const uint2*>(static_cast<const __half*>(in.ptr[a]) + off[a]));
              const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
              const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
              xa[0] = lo.x; xa[1 % V] = lo.y; xa[2 % V] = hi.x; xa[3 % V] = hi.y;
            }
          } else {
#pragma unroll
            for (int v = 0; v < V; ++v) xa[v] = load1<T>(in.ptr[a], off[a] + v * st0[a]);
          }
        } else {
#pragma unroll
          for (int v = 0; v < V; ++v) xa[v] = 0.f;
        }
      }
    }
    float s0[E], s1[ES], s2[ES], s3[ES];  // the stack, top (the accumulator) first
#pragma unroll
    for (int v = 0; v < E; ++v) s0[v] = 0.f;
#pragma unroll
    for (int v = 0; v < ES; ++v) s1[v] = s2[v] = s3[v] = 0.f;
    for (int k = 0; k < prog.n_ins; ++k) {
      const unsigned w = prog.ins[k];
      const unsigned kind = w & 3u, src = (w >> 2) & 3u, code = (w >> 8) & 0xffu, arg = (w >> 16) & 0xffu;
      if (kind == K_UNARY) {
        // one dispatch per instruction and thread, not per element
#define CTB_U(CODE, EXPR)               \
  case CODE:                            \
    _Pragma("unroll") for (int v = 0; v < E; ++v) { const float t = s0[v]; s0[v] = (EXPR); } \
    break;
        switch (code) {
          CTB_U(CTB_TILED_NEG, -t)
          CTB_U(CTB_TILED_ABS, fabsf(t))
          CTB_U(CTB_TILED_SQRT, sqrtf(t))
          CTB_U(CTB_TILED_EXP, expf(t))
          CTB_U(CTB_TILED_EXP2, exp2f(t))
          CTB_U(CTB_TILED_LOG, logf(t))
          CTB_U(CTB_TILED_LOG2, log2f(t))
          CTB_U(CTB_TILED_SIN, sinf(t))
          CTB_U(CTB_TILED_COS, cosf(t))
          CTB_U(CTB_TILED_TANH, tanhf(t))
          CTB_U(CTB_TILED_INV, 1.0f / t)
          CTB_U(CTB_TILED_ABS2, t * t)
          default: break;
        }
#undef CTB_U
        continue;
      }
      float t[E];  // the operand
      if (src == SRC_INPUT) {
        const unsigned which = NIN == 1 ? 0u : NIN == 2 ? (arg & 1u) : (arg & 3u);
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
          if (which == (unsigned)a) {
#pragma unroll
            for (int v = 0; v < E; ++v) t[v] = x[a][v];
          }
        }
      } else if (src == SRC_CONST) {
        const float c = prog.consts[arg & (kMaxConsts - 1)];
#pragma unroll
        for (int v = 0; v < E; ++v) t[v] = c;
      } else {  // the entry below the accumulator, popped (DEEP programs only)
#pragma unroll
        for (int v = 0; v < E; ++v) {
          t[v] = s1[v % ES];
          if (DEEP) { s1[v % ES] = s2[v % ES]; s2[v % ES] = s3[v % ES]; }
        }
      }
      if (kind == K_LOAD) {
#pragma unroll
        for (int v = 0; v < E; ++v) {
          if (DEEP) { s3[v % ES] = s2[v % ES]; s2[v % ES] = s1[v % ES]; s1[v % ES] = s0[v]; }
          s0[v] = t[v];
        }
        continue;
      }
      if (w & kRevBit) {
#pragma unroll
        for (int v = 0; v < E; ++v) {
          const float q = s0[v]; s0[v] = t[v]; t[v] = q;
        }
      }
#define CTB_B(CODE, EXPR)               \
  case CODE:                            \
    _Pragma("unroll") for (int v = 0; v < E; ++v) { const float a = s0[v], b = t[v]; s0[v] = (EXPR); } \
    break;
      switch (code) {
        CTB_B(CTB_TILED_ADD, a + b)
        CTB_B(CTB_TILED_SUB, a - b)
        CTB_B(CTB_TILED_MUL, a * b)
        CTB_B(CTB_TILED_DIV, a / b)
        CTB_B(CTB_TILED_MAX, fmaxf(a, b))
        CTB_B(CTB_TILED_MIN, fminf(a, b))
        default:
#pragma unroll
          for (int v = 0; v < E; ++v) s0[v] = powf(s0[v], t[v]);
          break;
      }
#undef CTB_B
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!live[g]) continue;
      const float* r = &s0[g * V];
      if (V == 4) {
        if constexpr (sizeof(T) == 4) {
          __stcs(reinterpret_cast<float4*>(static_cast<float*>(dest) + o[g]), make_float4(r[0], r[1 % V], r[2 % V], r[3 % V]));
        } else {
          uint2 q;
          *reinterpret_cast<__half2*>(&q.x) = __floats2half2_rn(r[0], r[1 % V]);
          *reinterpret_cast<__half2*>(&q.y) = __floats2half2_rn(r[2 % V], r[3 % V]);
          __stcs(reinterpret_cast<uint2*>(static_cast<__half*>(dest) + o[g]), q);
        }
      } else {
        store1<T>(dest, o[g], r[0]);
      }
    }
  }
}

// ---- sine and cosine for the vector path ---------------------------------------------------------------------------
// The library's sinf / cosf test every element for a huge argument and branch; for a thread's 4 * G elements that
// is most of the instructions of a short expression.  Here the test is made once for all of a thread's elements and
// the common case runs without a branch:  j = round(|x| * 2/pi) by the magic-number addition, r = |x| - j * pi/2 with
// pi/2 split in three f32 parts (every step one FMA; for |x| <= 105615 the first difference is exact), then
// sin(r) = r + r s (S0 + S1 s + S2 s^2) or cos(r) = 1 - s/2 + s^2 (C0 + C1 s + C2 s^2) with s = r^2, picked by the
// parity of j, the sign by bit 1 of j (and by the sign of x for the sine, which keeps sin(-0) = -0).  The
// coefficients are a weighted minimax fit on |r| <= pi/4 (fit errors 3.6e-9 relative and 9.6e-11).  The same
// arithmetic evaluated on a CPU for every f32 in [0, 105615] differs from the exact value by at most 1.54 ulp
// (0.02 % of the arguments by more than 1 ulp).  Anything larger, infinite or NaN takes sinf / cosf.
constexpr float kSinCosLimit = 105615.0f;
template <bool COS>
__device__ __forceinline__ float sincos_reduced(float x) {
  constexpr float kTwoOverPi = 0.636619772367581343f, kMagic = 12582912.0f;  // 1.5 * 2^23
  constexpr float P1 = 0x1.921fb6p+0f, P2 = -0x1.777a5cp-25f, P3 = -0x1.ee59dap-50f;  // sum = pi/2 to 2^-74
  constexpr float S0 = -0.16666655242443085f, S1 = 0.008332176133990288f, S2 = -0.00019516977772582322f;
  constexpr float C0 = 0.04166664555668831f, C1 = -0.0013887364184483886f, C2 = 2.443809171381872e-05f;
  const float ax = fabsf(x);
  float jf = __fmaf_rn(ax, kTwoOverPi, kMagic);
  unsigned q = __float_as_uint(jf);  // the low bits of the mantissa hold j
  jf = __fadd_rn(jf, -kMagic);
  float r = __fmaf_rn(jf, -P1, ax);
  r = __fmaf_rn(jf, -P2, r);
  r = __fmaf_rn(jf, -P3, r);
  if (COS) q += 1u;  // cos(x) = sin(x + pi/2)
  const float s = __fmul_rn(r, r);
  // both polynomials, one select: selects and bit operations issue at half the rate of FMAs
  float ps = __fmaf_rn(s, S2, S1);
  ps = __fmaf_rn(s, ps, S0);
  ps = __fmaf_rn(__fmul_rn(s, r), ps, r);
  float pc = __fmaf_rn(s, C2, C1);
  pc = __fmaf_rn(s, pc, C0);
  pc = __fmaf_rn(s, pc, -0.5f);
  pc = __fmaf_rn(s, pc, 1.0f);
  const float res = (q & 1u) ? pc : ps;
  unsigned sign = (q & 2u) << 30;
  if (!COS) sign ^= __float_as_uint(x) & 0x80000000u;
  return __uint_as_float(__float_as_uint(res) ^ sign);
}
template <bool COS, int E>
__device__ __forceinline__ void sincos_all(float (&a)[E]) {
  bool in_range = true;
#pragma unroll
  for (int v = 0; v < E; ++v) in_range = in_range && (fabsf(a[v]) <= kSinCosLimit);  // false for NaN
  if (in_range) {
#pragma unroll
    for (int v = 0; v < E; ++v) a[v] = sincos_reduced<COS>(a[v]);
  } else {
#pragma unroll
    for (int v = 0; v < E; ++v) a[v] = COS ? cosf(a[v]) : sinf(a[v]);
  }
}

// ---- the vector path: operands staged in shared memory by cp.async, two trips deep ----------------------------------
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
// 16 or 8 bytes global -> shared, asynchronous; src_bytes = 0 writes zeros and reads nothing
template <int BYTES>
__device__ __forceinline__ void cp_async_group(unsigned dst, const void* src, unsigned src_bytes) {
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The element-wise part of one instruction, for all of a thread's elements.  The operation, its direction and the
// kind of operand are template parameters and every instruction has its own straight-line code under the kernel's
// dispatch: with run-time tests on them around the element loops a multiplication by a constant executed 8.2
// instructions per element (counted with ncu by differencing programs), with straight-line code 4.5.
template <int CODE, bool REV>
__device__ __forceinline__ float binary_op(float p, float q) {
  const float a = REV ? q : p, b = REV ? p : q;
  if constexpr (CODE == CTB_TILED_ADD) return a + b;
  else if constexpr (CODE == CTB_TILED_SUB) return a - b;
  else if constexpr (CODE == CTB_TILED_MUL) return a * b;
  else if constexpr (CODE == CTB_TILED_DIV) return a / b;
  else if constexpr (CODE == CTB_TILED_MAX) return fmaxf(a, b);
  else if constexpr (CODE == CTB_TILED_MIN) return fminf(a, b);
  else return powf(a, b);
}
template <int CODE, bool REV, int E>
__device__ __forceinline__ void apply_binary(float (&s0)[E], const float (&t)[E]) {
#pragma unroll
  for (int v = 0; v < E; ++v) s0[v] = binary_op<CODE, REV>(s0[v], t[v]);
}
template <int CODE, bool REV, int E>
__device__ __forceinline__ void apply_binary(float (&s0)[E], float c) {
#pragma unroll
  for (int v = 0; v < E; ++v) s0[v] = binary_op<CODE, REV>(s0[v], c);
}
template <int CODE, int E>
__device__ __forceinline__ void apply_unary(float (&s0)[E]) {
  if constexpr (CODE == CTB_TILED_SIN) {
    sincos_all<false>(s0);
  } else if constexpr (CODE == CTB_TILED_COS) {
    sincos_all<true>(s0);
  } else {
#pragma unroll
    for (int v = 0; v < E; ++v) s0[v] = unary(CODE, s0[v]);  // CODE is a constant: the switch inside folds
  }
}

// Calls f(integral_constant<IDX>) for the run-time idx in [LO, HI) through a balanced tree of compares: six uniform
// branches for the 56 instructions (measured 4 % faster on a four-instruction program than a switch over the same cases).
template <unsigned LO, unsigned HI, typename F>
__device__ __forceinline__ void tree_dispatch(unsigned idx, F&& f) {
  if constexpr (HI - LO == 1) {
    f(std::integral_constant<unsigned, LO>());
  } else {
    constexpr unsigned MID = (LO + HI) / 2;
    if (idx < MID) tree_dispatch<LO, MID>(idx, f);
    else tree_dispatch<MID, HI>(idx, f);
  }
}
constexpr unsigned kDispatchCount = kDispatchBinary + 7 * 6;

// Every operand is contiguous along the first dimension with 16-byte aligned rows, or expanded along it (the host
// checks).  A group is four neighbouring elements; a thread owns G groups per trip, a whole grid apart.  The
// operands of the NEXT trip are copied global -> shared by cp.async (no registers, nothing waits on them) while the
// instructions run on the current trip's copies, so the latency of HBM is off the critical path whatever the
// occupancy; registers hold only the accumulator, the current operand and, for DEEP programs, the three stack
// entries.  A thread reads only the shared memory it filled itself: no CTA barrier anywhere.
// Shared memory: [2 buffers][n_inputs][G][256 threads] groups of 4 * sizeof(T) bytes.
// Addresses: with DENSE operands a thread keeps one running pointer per array and adds a trip's bytes to it; a trip
// whose G groups all exist (all but a thread's last) runs without a bounds test.
template <typename T, int G, bool DENSE, bool DEEP>
__global__ void __launch_bounds__(256)
    tiled_broadcast_pipe_kernel(void* __restrict__ dest, const Operands in, const Program prog, int n_inputs, long long d0,
                                long long d1, long long d2) {
  constexpr int V = 4, E = V * G, VB = V * (int)sizeof(T);
  constexpr int ES = DEEP ? E : 1;
  extern __shared__ __align__(16) unsigned char tiled_smem[];
  const long long n0 = d0 / V, total = n0 * d1 * d2;
  const long long grid_stride = (long long)gridDim.x * blockDim.x;
  const long long group_bytes = grid_stride * VB;  // from one of a thread's groups to the next, in a dense array
  const unsigned tid = threadIdx.x;
  const unsigned buf_bytes = (unsigned)n_inputs * G * 256 * VB;
  const unsigned smem0 = smem_addr(tiled_smem) + tid * VB;
  auto slot = [&](unsigned buf, unsigned a, unsigned g) { return smem0 + buf * buf_bytes + (a * G + g) * (256 * VB); };

  long long i = (long long)blockIdx.x * blockDim.x + tid;
  // running pointers (DENSE): this thread's first group of the trip to copy next / to store next
  const char* src_p[kMaxInputs];
#pragma unroll
  for (int a = 0; a < kMaxInputs; ++a) src_p[a] = static_cast<const char*>(in.ptr[a]) + i * VB;
  char* dst_p = static_cast<char*>(dest) + i * VB;

  // element offset of group ig in the destination (the general case)
  auto dest_offset = [&](long long ig) -> long long {
    const unsigned u = (unsigned)ig, un0 = (unsigned)n0, ud1 = (unsigned)d1;
    const unsigned r = u / un0, i0 = (u - r * un0) * V, i2 = r / ud1, i1 = r - i2 * ud1;
    return i0 + d0 * (i1 + d1 * (long long)i2);
  };
  auto issue = [&](long long at, unsigned buf, auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long ig = at + g * grid_stride;
      const bool live = FULL || ig < total;
      unsigned i0 = 0, i1 = 0, i2 = 0;
      if (!DENSE) {
        const unsigned u = live ? (unsigned)ig : 0u, un0 = (unsigned)n0, ud1 = (unsigned)d1;
        const unsigned r = u / un0;
        i0 = (u - r * un0) * V, i2 = r / ud1, i1 = r - i2 * ud1;
      }
#pragma unroll
      for (int a = 0; a < kMaxInputs; ++a) {
        if (a < n_inputs) {  // uniform
          const bool contiguous = in.stride[a][0] == 1;
          const char* src;
          if (DENSE) {
            src = contiguous ? src_p[a] + g * group_bytes : static_cast<const char*>(in.ptr[a]);
          } else {
            src = static_cast<const char*>(in.ptr[a]) +
                  (i0 * in.stride[a][0] + i1 * in.stride[a][1] + i2 * in.stride[a][2]) * (long long)sizeof(T);
          }
          if (contiguous) {
            if (FULL) cp_async_group<VB>(slot(buf, a, g), src, VB);
            else cp_async_group<VB>(slot(buf, a, g), live ? src : static_cast<const char*>(in.ptr[a]), live ? VB : 0);
          } else if (live) {  // expanded along the first dimension: one element, four copies
            const T v = *reinterpret_cast<const T*>(src);
            T* dst = reinterpret_cast<T*>(tiled_smem + (slot(buf, a, g) - smem_addr(tiled_smem)));
            dst[0] = v; dst[1] = v; dst[2] = v; dst[3] = v;
          }
        }
      }
    }
    if (DENSE) {
#pragma unroll
      for (int a = 0; a < kMaxInputs; ++a) src_p[a] += group_bytes * G;
    }
    cp_async_commit();
  };
  // the four elements of every group of operand `a`, from shared memory
  auto fetch = [&](unsigned buf, unsigned a, float (&t)[E]) {
    const unsigned base = slot(buf, a & (kMaxInputs - 1), 0);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if constexpr (sizeof(T) == 4) {
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(t[4 * g]), "=f"(t[4 * g + 1]), "=f"(t[4 * g + 2]), "=f"(t[4 * g + 3])
                     : "r"(base + g * (256 * VB)));
      } else {
        uint2 q;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "r"(base + g * (256 * VB)));
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
        t[4 * g] = lo.x; t[4 * g + 1] = lo.y; t[4 * g + 2] = hi.x; t[4 * g + 3] = hi.y;
      }
    }
  };
  auto start_next = [&](long long at, unsigned buf) {
    if (at + (G - 1) * grid_stride < total) issue(at, buf, std::true_type());
    else if (at < total) issue(at, buf, std::false_type());
    else cp_async_commit();  // an empty group keeps the count in the wait below uniform
  };

  start_next(i, 0);
  for (unsigned buf = 0; i < total; i += grid_stride * G, buf ^= 1u) {
    start_next(i + grid_stride * G, buf ^ 1u);
    cp_async_wait<1>();  // everything but the newest group has landed: this trip's operands

    float s0[E], s1[ES], s2[ES], s3[ES];  // the stack, top (the accumulator) first; every program starts with a push
#pragma unroll
    for (int v = 0; v < ES; ++v) s1[v] = s2[v] = s3[v] = 0.f;
    auto push = [&]() {
      if (DEEP) {
#pragma unroll
        for (int v = 0; v < ES; ++v) { s3[v] = s2[v]; s2[v] = s1[v]; s1[v] = s0[v % E]; }
      }
    };
    auto pop = [&](float (&t)[E]) {  // DEEP programs only
#pragma unroll
      for (int v = 0; v < E; ++v) {
        t[v] = s1[v % ES];
        if (DEEP) { s1[v % ES] = s2[v % ES]; s2[v % ES] = s3[v % ES]; }
      }
    };
    for (int k = 0; k < prog.n_ins; ++k) {
      const unsigned w = prog.ins[k];
      const unsigned arg = (w >> 16) & 0xffu;
      tree_dispatch<0, 64>(w >> 24, [&](auto tag) {
        constexpr unsigned IDX = decltype(tag)::value;
        if constexpr (IDX == 0) {
          push();
          fetch(buf, arg, s0);
        } else if constexpr (IDX == 1) {
          push();
          const float c = prog.consts[arg & (kMaxConsts - 1)];
#pragma unroll
          for (int v = 0; v < E; ++v) s0[v] = c;
        } else if constexpr (IDX < kDispatchBinary) {
          apply_unary<(int)(CTB_TILED_NEG + IDX - kDispatchUnary)>(s0);
        } else if constexpr (IDX < kDispatchCount) {
          constexpr unsigned VARIANT = (IDX - kDispatchBinary) / 7;
          constexpr int CODE = (int)(CTB_TILED_ADD + (IDX - kDispatchBinary) % 7);
          constexpr bool REV = VARIANT & 1u;
          if constexpr (VARIANT / 2 == 0) {  // an input
            float t[E];
            fetch(buf, arg, t);
            apply_binary<CODE, REV>(s0, t);
          } else if constexpr (VARIANT / 2 == 1) {  // a constant
            apply_binary<CODE, REV>(s0, prog.consts[arg & (kMaxConsts - 1)]);
          } else if constexpr (DEEP) {  // the entry below the accumulator
            float t[E];
            pop(t);
            apply_binary<CODE, REV>(s0, t);
          }
        }
      });
    }
    const bool full = i + (G - 1) * grid_stride < total;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!full && i + g * grid_stride >= total) continue;
      char* out = DENSE ? dst_p + g * group_bytes : static_cast<char*>(dest) + dest_offset(i + g * grid_stride) * (long long)sizeof(T);
      const float* r = &s0[g * V];
      if constexpr (sizeof(T) == 4) {
        __stcs(reinterpret_cast<float4*>(out), make_float4(r[0], r[1], r[2], r[3]));
      } else {
        uint2 q;
        *reinterpret_cast<__half2*>(&q.x) = __floats2half2_rn(r[0], r[1]);
        *reinterpret_cast<__half2*>(&q.y) = __floats2half2_rn(r[2], r[3]);
        __stcs(reinterpret_cast<uint2*>(out), q);
      }
    }
    dst_p += group_bytes * G;
  }
  cp_async_wait<0>();
}

template <typename T, int G, bool DENSE, bool DEEP>
int launch_pipe(ctb_ctx* ctx, cudaStream_t st, void* dest, const Operands& in, const Program& prog, int n_inputs, long long d0,
                long long d1, long long d2, long long units) {
  auto kernel = tiled_broadcast_pipe_kernel<T, G, DENSE, DEEP>;
  const int smem = std::max(1, n_inputs) * 2 * G * 256 * 4 * (int)sizeof(T);
  if (smem > 48 * 1024 &&  // per device, so on every launch that needs it: a host-side table write
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(CTB_CUDA_ERROR, "ctb_tiled_broadcast: shared memory attribute: %s", cudaGetErrorString(cudaGetLastError()));
  // Several waves of CTAs, not one wave of resident ones: CTAs that all start together stay in step (all loading,
  // then all storing) and measured 10 % slower than CTAs that start at different times.
  const long long ctas = (units + 256ll * G - 1) / (256ll * G);
  const int grid = (int)std::max<long long>(1, std::min<long long>(ctas, (long long)ctx->sm_count * 16));
  kernel<<<grid, 256, smem, st>>>(dest, in, prog, n_inputs, d0, d1, d2);
  return CTB_OK;
}

// ---- mapreduce ----------------------------------------------------------------------------------------------------
__device__ __forceinline__ float neutral(int op) {
  return op == CTB_TILED_ADD ? 0.f : op == CTB_TILED_MUL ? 1.f : op == CTB_TILED_MAX ? -INFINITY : INFINITY;
}

struct ReduceShape {
  long long d[3];        // extents
  long long keep_n[3];   // extent of each dimension in the output index space (1 when reduced)
  long long red_n[3];    // extent of each dimension in the reduced index space (1 when kept)
  long long outputs, red_len, parts, chunk;
};

// Mode A (the first dimension is reduced): one CTA per (output, part).  The reduced index space is the first
// dimension (contiguous) times the other reduced dimensions ("rows"); a part is a range [lo, hi) of it.  The CTA walks
// its rows one after the other, inside a row 16 bytes per thread and trip where the row starts on a 16-byte boundary,
// and combines in a fixed order (thread partials, lanes, then warps in order).
// Mode B (the first dimension is kept): one thread per output, outputs along the first dimension in neighbouring
// threads (coalesced), the part's share of the reduced index space walked in order with running coordinates.
// OP is a compile-time constant and so is "f is the identity": a dispatch per element would cost more than the element.
template <typename T, bool MODE_A, int OP, bool MAPPED, int VB = 1>
__global__ void __launch_bounds__(256)
    tiled_reduce_kernel(const void* __restrict__ src, float* __restrict__ partial, void* __restrict__ dest, const ReduceShape s,
                        int f_code) {
  constexpr int op = OP;
  auto fmap = [&](float v) { return MAPPED ? unary(f_code, v) : v; };
  __shared__ float wsum[8];
  const long long part = blockIdx.y;
  const long long lo = part * s.chunk, hi = min(s.red_len, lo + s.chunk);
  const long long st1 = s.d[0], st2 = s.d[0] * s.d[1];  // element strides of dimensions 1 and 2
  if (MODE_A) {
    // output coordinates: the first dimension is reduced, so the output index runs over dimensions 1 and 2
    const long long o = blockIdx.x;
    const long long k1 = o % s.keep_n[1], k2 = o / s.keep_n[1];
    const long long base = k1 * st1 + k2 * st2;
    const long long d0 = s.d[0];
    constexpr int V = 16 / sizeof(T);
    float acc = neutral(op);
    for (long long row = lo / d0; row * d0 < hi; ++row) {  // rows of the reduced index space that this part touches
      const long long r1 = row % s.red_n[1], r2 = row / s.red_n[1];
      const long long rbase = base + r1 * st1 + r2 * st2;
      const long long c_lo = max(lo - row * d0, 0ll), c_hi = min(hi - row * d0, d0);
      const bool vec = ((rbase + c_lo) * (long long)sizeof(T) + (long long)(uintptr_t)src) % 16 == 0;
      const long long c_vec = vec ? c_lo + (c_hi - c_lo) / V * V : c_lo;
      for (long long c = c_lo + (long long)threadIdx.x * V; c < c_vec; c += 256 * V) {
        if constexpr (sizeof(T) == 4) {
          const float4 q = __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(src) + rbase + c));
          acc = binary(op, acc, fmap(q.x));
          acc = binary(op, acc, fmap(q.y));
          acc = binary(op, acc, fmap(q.z));
          acc = binary(op, acc, fmap(q.w));
        } else {
          const uint4 q = __ldcs(reinterpret_cast<const uint4*>(static_cast<const __half*>(src) + rbase + c));
          const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 v = __half22float2(h[j]);
            acc = binary(op, acc, fmap(v.x));
            acc = binary(op, acc, fmap(v.y));
          }
        }
      }
      for (long long c = c_vec + threadIdx.x; c < c_hi; c += 256) acc = binary(op, acc, fmap(load1<T>(src, rbase + c)));
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) acc = binary(op, acc, __shfl_xor_sync(0xffffffffu, acc, sh));
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = wsum[0];
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) t = binary(op, t, wsum[w]);
      if (s.parts > 1) partial[o * s.parts + part] = t;
      else store1<T>(dest, o, t);
    }
  } else {
    // VB neighbouring outputs per thread (VB = 4: the first extent is a multiple of four and the rows start on
    // aligned boundaries, so the four outputs share their other coordinates and one 16-byte / 8-byte load fetches an
    // element of each); eight loads in flight per thread, combined in index order: the order of summation of every
    // output is the same as with one output per thread.
    const long long o = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VB;
    if (o >= s.outputs) return;
    // output coordinates over the kept dimensions (the first one is kept), reduced coordinates over dimensions 1 and 2
    const long long k0 = o % s.keep_n[0], q = o / s.keep_n[0], k1 = q % s.keep_n[1], k2 = q / s.keep_n[1];
    const long long base = k0 + k1 * st1 + k2 * st2;
    long long r1 = lo % s.red_n[1], r2 = lo / s.red_n[1];
    long long off = base + r1 * st1 + r2 * st2;
    auto advance = [&]() {  // to the next reduced coordinate, dimension 1 fastest
      off += st1;
      if (++r1 == s.red_n[1]) {
        r1 = 0;
        ++r2;
        off = base + r2 * st2;
      }
    };
    auto load = [&](long long at, float (&v)[VB]) {
      if constexpr (VB == 1) {
        v[0] = load1<T>(src, at);
      } else if constexpr (sizeof(T) == 4) {
        const float4 x = __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(src) + at));
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
      } else {
        const uint2 x = __ldcs(reinterpret_cast<const uint2*>(static_cast<const __half*>(src) + at));
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
      }
    };
    constexpr int kFlight = VB == 1 ? 4 : 8;
    float acc[VB];
#pragma unroll
    for (int e = 0; e < VB; ++e) acc[e] = neutral(op);
    long long r = lo;
    for (; r + kFlight <= hi; r += kFlight) {
      float v[kFlight][VB];
#pragma unroll
      for (int j = 0; j < kFlight; ++j) {
        load(off, v[j]);
        advance();
      }
#pragma unroll
      for (int j = 0; j < kFlight; ++j)
#pragma unroll
        for (int e = 0; e < VB; ++e) acc[e] = binary(op, acc[e], fmap(v[j][e]));
    }
    for (; r < hi; ++r) {
      float v[VB];
      load(off, v);
      advance();
#pragma unroll
      for (int e = 0; e < VB; ++e) acc[e] = binary(op, acc[e], fmap(v[e]));
    }
#pragma unroll
    for (int e = 0; e < VB; ++e) {
      if (s.parts > 1) partial[(o + e) * s.parts + part] = acc[e];
      else store1<T>(dest, o + e, acc[e]);
    }
  }
}

template <typename T, int OP>
__global__ void tiled_reduce_final_kernel(const float* __restrict__ partial, void* __restrict__ dest, long long outputs,
                                          long long parts) {
  constexpr int op = OP;
  const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= outputs) return;
  float acc = partial[o * parts];
  for (long long p = 1; p < parts; ++p) acc = binary(op, acc, partial[o * parts + p]);  // ascending part order
  store1<T>(dest, o, acc);
}

}  // namespace

extern "C" {

int ctb_tiled_broadcast(ctb_ctx* ctx, void* stream, void* dest, const int64_t* shape, const void* const* inputs,
                        const int64_t* input_strides, int n_inputs, const int32_t* program, int n_ops, const float* constants,
                        int n_constants, int dtype) {
  CTB_CHECK_CTX(ctx);
  if (!shape || !program) return fail(CTB_BAD_ARG, "ctb_tiled_broadcast: null shape or program");
  if (dtype != CTB_F32 && dtype != CTB_F16) return fail(CTB_UNSUPPORTED, "ctb_tiled_broadcast: element type must be f32 or f16");
  if (n_inputs < 0 || n_inputs > kMaxInputs || n_ops < 1 || n_ops > kMaxOps || n_constants < 0 || n_constants > kMaxConsts)
    return fail(CTB_UNSUPPORTED, "ctb_tiled_broadcast: at most %d inputs, %d operations and %d constants", kMaxInputs, kMaxOps,
                kMaxConsts);
  if ((n_inputs && (!inputs || !input_strides)) || (n_constants && !constants))
    return fail(CTB_BAD_ARG, "ctb_tiled_broadcast: null operand table");
  for (int k = 0; k < 3; ++k)
    if (shape[k] < 0) return fail(CTB_BAD_ARG, "ctb_tiled_broadcast: negative extent");
  Program prog;
  const char* why = "";
  int need = 1;
  const int bad = compile_program(program, n_ops, n_inputs, n_constants, &prog, &why, &need);
  if (bad == -1000)
    return fail(CTB_UNSUPPORTED, "ctb_tiled_broadcast: the expression needs more than %d intermediate values at once", kStack);
  if (bad) return fail(CTB_BAD_ARG, "ctb_tiled_broadcast: operation %d %s", -bad - 1, why);
  for (int k = 0; k < n_constants; ++k) prog.consts[k] = constants[k];
  const long long d0 = shape[0], d1 = shape[1], d2 = shape[2];
  if (d0 == 0 || d1 == 0 || d2 == 0) return CTB_OK;  // empty arrays: nothing to launch
  CTB_CHECK_DEV(dest);
  const int es = dtype == CTB_F32 ? 4 : 2;
  Operands in = {};
  bool vec = d0 % 4 == 0 && (uintptr_t)dest % 16 == 0;
  for (int a = 0; a < n_inputs; ++a) {
    CTB_CHECK_DEV(inputs[a]);
    in.ptr[a] = inputs[a];
    for (int k = 0; k < 3; ++k) {
      in.stride[a][k] = input_strides[3 * a + k];
      if (in.stride[a][k] < 0) return fail(CTB_BAD_ARG, "ctb_tiled_broadcast: negative stride");
    }
    const long long s0 = in.stride[a][0];
    if (s0 == 1) {  // vector loads need aligned rows
      if ((uintptr_t)inputs[a] % (4 * es) || (in.stride[a][1] * es) % (4 * es) || (in.stride[a][2] * es) % (4 * es)) vec = false;
    } else if (s0 != 0) {
      vec = false;
    }
  }
  // dense: every operand is laid out like the destination or is a single element
  bool dense = true;
  for (int a = 0; a < n_inputs; ++a) {
    const bool like_dest = in.stride[a][0] == 1 && (d1 == 1 || in.stride[a][1] == d0) && (d2 == 1 || in.stride[a][2] == d0 * d1);
    const bool single = in.stride[a][0] == 0 && (d1 == 1 || in.stride[a][1] == 0) && (d2 == 1 || in.stride[a][2] == 0);
    if (!like_dest && !single) dense = false;
  }
  const long long units = (vec ? d0 / 4 : d0) * d1 * d2;
  if (!dense && units > 0x7fffffffLL) return fail(CTB_UNSUPPORTED, "ctb_tiled_broadcast: too many elements for an expanded operand");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool deep = need > 1;
  int rc = CTB_OK;
  // groups per thread: as many as registers (the stack of a deep program) and shared memory (the operands) allow;
  // eight groups for a single operand measured slower than four (128 registers, two CTAs per SM)
#define CTB_TILED_VEC(T, D)                                                                                          \
  do {                                                                                                               \
    if (deep) rc = launch_pipe<T, 2, D, true>(ctx, st, dest, in, prog, n_inputs, d0, d1, d2, units);                 \
    else if (n_inputs <= 3) rc = launch_pipe<T, 4, D, false>(ctx, st, dest, in, prog, n_inputs, d0, d1, d2, units);  \
    else rc = launch_pipe<T, 2, D, false>(ctx, st, dest, in, prog, n_inputs, d0, d1, d2, units);                     \
  } while (0)
#define CTB_TILED_SCALAR(T, D)                                                                                       \
  do {                                                                                                               \
    const int grid = (int)std::max<long long>(1, std::min<long long>((units + 255) / 256, (long long)ctx->sm_count * 16)); \
    tiled_broadcast_kernel<T, 1, 1, D, kMaxInputs, true><<<grid, 256, 0, st>>>(dest, in, prog, n_inputs, d0, d1, d2); \
  } while (0)
#define CTB_TILED_PICK(T)                                                     \
  do {                                                                        \
    if (vec && dense) CTB_TILED_VEC(T, true);                                 \
    else if (vec) CTB_TILED_VEC(T, false);                                    \
    else if (dense) CTB_TILED_SCALAR(T, true);                                \
    else CTB_TILED_SCALAR(T, false);                                          \
  } while (0)
  if (dtype == CTB_F32) CTB_TILED_PICK(float);
  else CTB_TILED_PICK(__half);
#undef CTB_TILED_PICK
#undef CTB_TILED_SCALAR
#undef CTB_TILED_VEC
  if (rc) return rc;
  CTB_CHECK_LAUNCH("ctb_tiled_broadcast launch");
  return CTB_OK;
}

int ctb_tiled_compile(const int32_t* program, int n_ops, int n_inputs, int n_constants, uint32_t* instructions,
                      int* n_instructions) {
  if (!program || !instructions || !n_instructions) return fail(CTB_BAD_ARG, "ctb_tiled_compile: null argument");
  if (n_inputs < 0 || n_inputs > kMaxInputs || n_ops < 1 || n_ops > kMaxOps || n_constants < 0 || n_constants > kMaxConsts)
    return fail(CTB_UNSUPPORTED, "ctb_tiled_compile: at most %d inputs, %d operations and %d constants", kMaxInputs, kMaxOps,
                kMaxConsts);
  Program prog;
  const char* why = "";
  const int bad = compile_program(program, n_ops, n_inputs, n_constants, &prog, &why);
  if (bad == -1000)
    return fail(CTB_UNSUPPORTED, "ctb_tiled_compile: the expression needs more than %d intermediate values at once", kStack);
  if (bad) return fail(CTB_BAD_ARG, "ctb_tiled_compile: operation %d %s", -bad - 1, why);
  for (int k = 0; k < prog.n_ins; ++k) instructions[k] = prog.ins[k];
  *n_instructions = prog.n_ins;
  return CTB_OK;
}

int ctb_tiled_mapreduce(ctb_ctx* ctx, void* stream, void* dest, const void* src, const int64_t* shape, int reduce_mask, int f,
                        int op, int dtype) {
  CTB_CHECK_CTX(ctx);
  if (!shape) return fail(CTB_BAD_ARG, "ctb_tiled_mapreduce: null shape");
  if (dtype != CTB_F32 && dtype != CTB_F16) return fail(CTB_UNSUPPORTED, "ctb_tiled_mapreduce: element type must be f32 or f16");
  if (f < CTB_TILED_IDENTITY || f > CTB_TILED_ABS2) return fail(CTB_BAD_ARG, "ctb_tiled_mapreduce: f must be a unary function code");
  if (op != CTB_TILED_ADD && op != CTB_TILED_MUL && op != CTB_TILED_MAX && op != CTB_TILED_MIN)
    return fail(CTB_UNSUPPORTED, "ctb_tiled_mapreduce: the reduction must be +, *, max or min");
  if (reduce_mask < 0 || reduce_mask > 7) return fail(CTB_BAD_ARG, "ctb_tiled_mapreduce: reduce_mask has bits for three dimensions");
  ReduceShape s;
  s.outputs = 1;
  s.red_len = 1;
  for (int k = 0; k < 3; ++k) {
    if (shape[k] < 0) return fail(CTB_BAD_ARG, "ctb_tiled_mapreduce: negative extent");
    s.d[k] = shape[k];
    const bool red = (reduce_mask >> k) & 1;
    s.keep_n[k] = red ? 1 : shape[k];
    s.red_n[k] = red ? shape[k] : 1;
    s.outputs *= s.keep_n[k];
    s.red_len *= s.red_n[k];
  }
  if (s.outputs == 0) return CTB_OK;  // no output elements
  CTB_CHECK_DEV(dest);
  if (s.red_len > 0) CTB_CHECK_DEV(src);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool mode_a = (reduce_mask & 1) != 0 && s.red_len > 0;
  // enough (output, part) pairs to fill the GPU; a part is at least 4096 reduced elements for a CTA, 32 for a thread
  const long long want = mode_a ? (long long)ctx->sm_count * 8 : (long long)ctx->sm_count * 8 * 256;
  const long long min_part = mode_a ? 4096 : 32;
  // first dimension kept: four neighbouring outputs per thread where 16-byte (f16: 8-byte) loads are aligned
  const int es = dtype == CTB_F32 ? 4 : 2;
  const int vb = (!mode_a && (reduce_mask & 1) == 0 && s.d[0] % 4 == 0 && (uintptr_t)src % (4 * es) == 0) ? 4 : 1;
  const long long work_items = mode_a ? s.outputs : s.outputs / vb;
  s.parts = std::max<long long>(1, std::min<long long>({want / std::max<long long>(1, work_items),
                                                        (s.red_len + min_part - 1) / min_part, (long long)1024}));
  s.chunk = (std::max<long long>(1, s.red_len) + s.parts - 1) / s.parts;
  if (mode_a) s.chunk = (s.chunk + 1023) / 1024 * 1024;  // parts start on 16-byte boundaries of an aligned row
  s.parts = (std::max<long long>(1, s.red_len) + s.chunk - 1) / s.chunk;
  float* partial = nullptr;
  if (s.parts > 1) {
    void* ws = nullptr;
    int r = workspace(ctx, (size_t)s.outputs * s.parts * sizeof(float), &ws, st);
    if (r) return r;
    partial = static_cast<float*>(ws);
  }
  if (mode_a && s.outputs > 0x7fffffffLL) return fail(CTB_UNSUPPORTED, "ctb_tiled_mapreduce: too many output elements");
  const dim3 grid(mode_a ? (unsigned)s.outputs : (unsigned)((work_items + 255) / 256), (unsigned)s.parts);
  const unsigned fgrid = (unsigned)((s.outputs + 255) / 256);
  const bool mapped = f != CTB_TILED_IDENTITY;
#define CTB_RED_LAUNCH(T, A, OP, M)                                                                \
  do {                                                                                             \
    if (!A && vb == 4) tiled_reduce_kernel<T, false, OP, M, 4><<<grid, 256, 0, st>>>(src, partial, dest, s, f); \
    else tiled_reduce_kernel<T, A, OP, M><<<grid, 256, 0, st>>>(src, partial, dest, s, f);        \
    if (s.parts > 1) tiled_reduce_final_kernel<T, OP><<<fgrid, 256, 0, st>>>(partial, dest, s.outputs, s.parts); \
  } while (0)
#define CTB_RED_MAPPED(T, A, OP)              \
  do {                                        \
    if (mapped) CTB_RED_LAUNCH(T, A, OP, true); \
    else CTB_RED_LAUNCH(T, A, OP, false);     \
  } while (0)
#define CTB_RED_OP(T, A)                                              \
  do {                                                                \
    if (op == CTB_TILED_ADD) CTB_RED_MAPPED(T, A, CTB_TILED_ADD);     \
    else if (op == CTB_TILED_MUL) CTB_RED_MAPPED(T, A, CTB_TILED_MUL); \
    else if (op == CTB_TILED_MAX) CTB_RED_MAPPED(T, A, CTB_TILED_MAX); \
    else CTB_RED_MAPPED(T, A, CTB_TILED_MIN);                         \
  } while (0)
  if (dtype == CTB_F32) {
    if (mode_a) CTB_RED_OP(float, true);
    else CTB_RED_OP(float, false);
  } else {
    if (mode_a) CTB_RED_OP(__half, true);
    else CTB_RED_OP(__half, false);
  }
#undef CTB_RED_OP
#undef CTB_RED_MAPPED
#undef CTB_RED_LAUNCH
  CTB_CHECK_LAUNCH("ctb_tiled_mapreduce launch");
  return CTB_OK;
}

}  // extern "C"
