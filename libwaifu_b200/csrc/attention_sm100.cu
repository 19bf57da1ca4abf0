// Scaled dot product attention on sm_100a. Two kernels: the one described first, one tile of
// queries per CTA, serves runs of at most 128 queries and the block diagonal mask; the two-tile
// kernel further down (probabilities in tensor memory, v read as it lies) serves the rest.
//
// A CTA owns 128 queries of one head and walks that head's keys 128 at a time. Per block of keys:
//   S = Q K^T      tcgen05.mma kind::f16, 128 x 128 x head_dim, into one of two score buffers in
//                  tensor memory (the next block's product runs beside this block's softmax);
//   softmax        eight warps, two threads per query (each half of the block's keys): a thread
//                  reads its part of the row of S from tensor memory (a row is a lane, so no
//                  shuffles; the two halves' maxima meet through shared memory), keeps the running
//                  maximum and its half of the sum, and writes P = exp2(S' - max) as 16-bit values
//                  into shared memory in the layout the next product reads its A operand in
//                  (128-byte swizzle, K-major);
//   O += P V       tcgen05.mma, 128 x head_dim x 128, accumulating in tensor memory; when a row's
//                  maximum has grown enough to matter the threads rescale their output rows
//                  there (tcgen05.ld / st) before handing P over.
// K and V blocks arrive by TMA into two-stage rings. V is the B operand of the second product and
// is read K-major, i.e. as V^T: a small kernel transposes it into scratch first.
//
// The arithmetic follows flint/cuda/attention.cu:30-70 (scores scaled by log2(e)/sqrt(head_dim)
// into exp2, float maximum, sum and output, 16-bit probabilities into the second product).
//
// Every wait is bounded: a role that gives up raises the CTA's abort flag, records a status word
// and the CTA leaves through the common teardown with its tensor memory freed.

#include "attention_sm100.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kBlockQ = 128;   // queries per CTA = lanes of tensor memory
constexpr int kBlockKv = 128;  // keys per step
constexpr int kAtomBytes = 128;  // one swizzle atom: 64 16-bit elements of K
constexpr int kAtomElems = 64;
constexpr int kMmaKBytes = 32;   // one kind::f16 instruction: 16 elements of K
constexpr int kSoftmaxWarps = 8;  // two per 32 queries
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 10 * 32;
constexpr int kKvStages = 2;
constexpr int kPadKv = 64;  // the transposed v's rows are padded to whole swizzle atoms

// Barriers and the exchange buffers sit behind the tiles in dynamic shared memory, so that the
// tiles start at the CTA's first byte, which is 1024-byte aligned (checked at entry).
struct Tail {
  uint64_t q_full_bar;
  uint64_t k_full_bar[kKvStages], k_empty_bar[kKvStages];
  uint64_t v_full_bar[kKvStages], v_empty_bar[kKvStages];
  uint64_t s_full_bar[2], s_empty_bar[2];  // the two score buffers
  uint64_t p_full_bar;                     // softmax -> MMA: the probabilities are in shared memory
  // MMA -> softmax: the block is in the output and its P buffer is free. One barrier per P buffer:
  // the softmax runs up to two products ahead of the one it waits for, and a waiter may lag an
  // mbarrier by less than two phases.
  uint64_t pv_done_bar[2];
  uint64_t pair_bar[4];  // the two warps that share 32 rows have both written their halves' maxima
  uint32_t tmem_base_slot;
  uint32_t abort_flag;
  float pair_value[2][2][kBlockQ];  // [block parity][column half][row]
};

template <int D>
struct Layout {
  static constexpr int kQAtoms = D / kAtomElems;                  // atoms along head_dim
  static constexpr int kQBytes = kQAtoms * kBlockQ * kAtomBytes;  // 128 rows x head_dim
  static constexpr int kKBytes = kQAtoms * kBlockKv * kAtomBytes;
  static constexpr int kVAtoms = kBlockKv / kAtomElems;           // atoms along the keys
  static constexpr int kVAtomBytes = D * kAtomBytes;              // head_dim rows x 64 keys
  static constexpr int kVBytes = kVAtoms * kVAtomBytes;
  static constexpr int kPAtomBytes = kBlockQ * kAtomBytes;
  static constexpr int kPBytes = kVAtoms * kPAtomBytes;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + kKvStages * kKBytes;
  static constexpr int kPOff = kVOff + kKvStages * kVBytes;
  static constexpr int kPBuffers = 2;  // the softmax of block j + 1 writes beside the product that reads block j's
  static constexpr int kTailOff = kPOff + kPBuffers * kPBytes;
  static constexpr int kSmemBytes = kTailOff + static_cast<int>(sizeof(Tail));
  // Tensor memory: two score buffers, then the block's output.
  static constexpr int kSCols = kBlockKv;
  static constexpr int kOCol = 2 * kSCols;
  static constexpr int kTmemCols = 512;
  static_assert(kOCol + D <= kTmemCols, "tensor memory holds 512 columns");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory");
};

struct KernelParams {
  void *out;
  int64_t out_stride[3];
  int is_bf16;
  int heads, group;  // group = heads / kv_heads
  int kv_heads;
  int q_len, kv_len;
  int mask_type;   // 0 none, 1 causal, 2 block causal, 3 block diagonal (flint/capi.h:118-133)
  int block_size;
  float scale_log2;
  int v_direct;  // two-tile kernel: v is read as it lies (an MN-major operand), not through its transposition
  uint32_t *status;
};

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *desc, uint64_t *bar, int32_t c0,
                                            int32_t c1, int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *desc, uint64_t *bar, int32_t c0,
                                            int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// The first and the last key a query at `position` may see (flint/cuda/attention.cu:165-179).
__device__ __forceinline__ int first_key_of(const KernelParams &p, int position) {
  return p.mask_type == 3 ? (position / p.block_size) * p.block_size : 0;
}
__device__ __forceinline__ int last_key_of(const KernelParams &p, int position) {
  if (p.mask_type == 0) return p.kv_len - 1;
  if (p.mask_type == 1) return min(p.kv_len - 1, position);
  return min(p.kv_len - 1, (position / p.block_size) * p.block_size + p.block_size - 1);
}

// 2^x for x <= 2^kRescaleStep's exponent: the hardware approximation (relative error 2^-22), -inf -> 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two floats in one 64-bit register, for the two-wide float instructions of sm_100.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float *lo, float *hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 2^x for a pair of exponents x <= 2^kRescaleStep's, without the special-function unit: that unit
// delivers 16 results a cycle and SM, so the 128 x 128 exponentials of a block would hold it for
// 1024 cycles; one pair in four of a row goes through here instead, on the multiply-add pipes
// (with one softmax warp per scheduler at work at a time, more than that costs more issue slots
// than it frees special-function cycles).
// x = n + f with n = round(x) (the low mantissa bits of x + 1.5 * 2^23) and f in [-0.5, 0.5]; 2^f
// by a cubic (relative error 7.5e-5, below the 16-bit rounding the probabilities get); n added
// into the exponent field. Exponents below -126 (masked keys are -inf) give 2^-126 or 0.
__device__ __forceinline__ void exp2_pair_poly(uint64_t x, float *e0, float *e1) {
  float x0, x1;
  f2_unpack(x, &x0, &x1);
  x = f2_pack(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
  const uint64_t t = f2_add(x, f2_pack(12582912.0f, 12582912.0f));
  const uint64_t n = f2_add(t, f2_pack(-12582912.0f, -12582912.0f));
  const uint64_t f = f2_fma(n, f2_pack(-1.0f, -1.0f), x);
  uint64_t q = f2_fma(f, f2_pack(0.05517162f, 0.05517162f), f2_pack(0.24261113f, 0.24261113f));
  q = f2_fma(q, f, f2_pack(0.69326097f, 0.69326097f));
  q = f2_fma(q, f, f2_pack(0.99992806f, 0.99992806f));
  float q0, q1, t0, t1;
  f2_unpack(q, &q0, &q1);
  f2_unpack(t, &t0, &t1);
  *e0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  *e1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// max(a, b, c) in one instruction.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ uint32_t pack16(float a, float b, int is_bf16) {
  if (is_bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// v (batch, kv_heads, kv_len, d) with strides -> vt (batch * kv_heads, d, kv_pad), zeros past kv_len.
// 64 x 64 tiles through shared memory; both sides coalesced.
__global__ void __launch_bounds__(256) transpose_v_kernel(const uint16_t *__restrict__ v, int64_t sb, int64_t sh,
                                                          int64_t sl, int kv_heads, int kv_len, int kv_pad, int d,
                                                          uint16_t *__restrict__ vt) {
  __shared__ uint16_t tile[64][66];
  const int bh = blockIdx.z;
  const int b = bh / kv_heads, h = bh % kv_heads;
  const int l0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const uint16_t *src = v + b * sb + h * sh;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int r = ty; r < 64; r += 4) {
    const int l = l0 + r;
    tile[r][tx] = (l < kv_len) ? src[static_cast<int64_t>(l) * sl + d0 + tx] : static_cast<uint16_t>(0);
  }
  __syncthreads();
  uint16_t *dst = vt + static_cast<int64_t>(bh) * d * kv_pad;
  for (int r = ty; r < 64; r += 4) {
    const int l = l0 + tx;
    if (l < kv_pad) dst[static_cast<int64_t>(d0 + r) * kv_pad + l] = tile[tx][r];
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_vt, const KernelParams p) {
  using L = Layout<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  Tail &t = *reinterpret_cast<Tail *>(smem + L::kTailOff);
  volatile uint32_t &abort_flag = *reinterpret_cast<volatile uint32_t *>(&t.abort_flag);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need it; uniform over the grid
    if (threadIdx.x == 0) atomicCAS(p.status, 0u, kStatusAttentionLayout);
    return;
  }
  const int q0 = static_cast<int>(p.mask_type != 0 ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * kBlockQ;  // longest walks first
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int offset = p.kv_len - p.q_len;  // query i sits at key position i + offset
  // The keys this CTA's queries can see between them: both ends of a query's range grow with its
  // position, so the range of the CTA runs from its first query's first key to its last query's
  // last key. Blocks of 128 keys outside it are never loaded.
  const int last_row = min(q0 + kBlockQ, p.q_len) - 1;
  const int kv_begin = first_key_of(p, q0 + offset);
  const int kv_end = last_key_of(p, last_row + offset) + 1;
  const int block0 = kv_begin / kBlockKv;  // first block of keys this CTA walks
  const int num_blocks = (kv_end + kBlockKv - 1) / kBlockKv - block0;

  if (threadIdx.x == 0) {
    t.abort_flag = 0;
    mbar_init(&t.q_full_bar, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&t.k_full_bar[s], 1);
      mbar_init(&t.k_empty_bar[s], 1);
      mbar_init(&t.v_full_bar[s], 1);
      mbar_init(&t.v_empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&t.s_full_bar[s], 1);
      mbar_init(&t.s_empty_bar[s], kSoftmaxWarps);
      mbar_init(&t.pv_done_bar[s], 1);
    }
    mbar_init(&t.p_full_bar, kSoftmaxWarps);
    for (int s = 0; s < 4; ++s) mbar_init(&t.pair_bar[s], 2);
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_vt);
  }
  if (warp == kMmaWarp) {
    tmem_alloc<1>(&t.tmem_base_slot, L::kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = t.tmem_base_slot;

  uint8_t *q_smem = smem + L::kQOff;
  auto k_stage = [&](int s) { return smem + L::kKOff + s * L::kKBytes; };
  auto v_stage = [&](int s) { return smem + L::kVOff + s * L::kVBytes; };
  uint8_t *p_smem = smem + L::kPOff;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      mbar_arrive_expect_tx(&t.q_full_bar, L::kQBytes);
#pragma unroll
      for (int a = 0; a < L::kQAtoms; ++a) {
        tma_load_4d(q_smem + a * kBlockQ * kAtomBytes, &tmap_q, &t.q_full_bar, a * kAtomBytes, q0, head, batch);
      }
      // K runs ahead of V: the scores of block j + 2 are multiplied beside P V of block j.
      auto load_k = [&](int j) -> bool {
        const int st = j % kKvStages;
        if (!mbar_wait(&t.k_empty_bar[st], ((j / kKvStages) & 1) ^ 1, &abort_flag)) return false;
        mbar_arrive_expect_tx(&t.k_full_bar[st], L::kKBytes);
#pragma unroll
        for (int a = 0; a < L::kQAtoms; ++a) {
          tma_load_4d(k_stage(st) + a * kBlockKv * kAtomBytes, &tmap_k, &t.k_full_bar[st], a * kAtomBytes, (block0 + j) * kBlockKv,
                      kv_head, batch);
        }
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int st = j % kKvStages;
        if (!mbar_wait(&t.v_empty_bar[st], ((j / kKvStages) & 1) ^ 1, &abort_flag)) return false;
        mbar_arrive_expect_tx(&t.v_full_bar[st], L::kVBytes);
#pragma unroll
        for (int a = 0; a < L::kVAtoms; ++a) {
          tma_load_3d(v_stage(st) + a * L::kVAtomBytes, &tmap_vt, &t.v_full_bar[st],
                      ((block0 + j) * kBlockKv + a * kAtomElems) * 2, 0, batch * p.kv_heads + kv_head);
        }
        return true;
      };
      ok = load_k(0);
      if (ok && num_blocks > 1) ok = load_k(1);
      for (int j = 0; j < num_blocks && ok; ++j) {
        ok = load_v(j);
        if (ok && j + 2 < num_blocks) ok = load_k(j + 2);
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusAttentionTimeout);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = umma_idesc(kBlockQ, kBlockKv, fmt, fmt);
      const uint32_t idesc_o = umma_idesc(kBlockQ, D, fmt, fmt);
      const uint64_t qdesc0 = umma_desc_sw128(smem_u32(q_smem));
      const uint64_t pdesc0 = umma_desc_sw128(smem_u32(p_smem));
      constexpr uint64_t kMmaStep = kMmaKBytes >> 4;
      constexpr int kMmasPerAtom = kAtomBytes / kMmaKBytes;
      constexpr int kScoreMmas = L::kQAtoms * kMmasPerAtom;  // per block
      constexpr int kOutMmas = L::kVAtoms * kMmasPerAtom;
      bool ok = true;
      // Everything an instruction needs is a per-parity base (stage, score buffer and P buffer all
      // alternate with the block index) plus a compile-time offset, so that the single issuing
      // thread spends its time on the instructions. (kind::f16 covers half and bfloat16: the
      // instruction descriptor carries the format.)
      static_assert(kKvStages == 2, "the stage of block j is j & 1");
      const uint64_t kdesc_0 = umma_desc_sw128(smem_u32(k_stage(0))), kdesc_1 = umma_desc_sw128(smem_u32(k_stage(1)));
      const uint64_t vdesc_0 = umma_desc_sw128(smem_u32(v_stage(0))), vdesc_1 = umma_desc_sw128(smem_u32(v_stage(1)));
      const uint64_t pdesc_1 = pdesc0 + (L::kPBytes >> 4);
      const uint32_t o_tmem = tmem_base + L::kOCol;
      // Instruction i of S = Q K^T (into the score buffer at s_tmem) and of O += P V.
      auto score_mma = [&](uint32_t s_tmem, uint64_t kd, int i) {
        const int a = i / kMmasPerAtom, s = i % kMmasPerAtom;
        umma_ss<kKindF16>(s_tmem, qdesc0 + (((a * kBlockQ * kAtomBytes) >> 4) + s * kMmaStep),
                          kd + (((a * kBlockKv * kAtomBytes) >> 4) + s * kMmaStep), idesc_s, i != 0 ? 1u : 0u);
      };
      auto out_mma = [&](uint64_t pd, uint64_t vd, int i, uint32_t first_block) {
        const int a = i / kMmasPerAtom, s = i % kMmasPerAtom;
        umma_ss<kKindF16>(o_tmem, pd + (((a * L::kPAtomBytes) >> 4) + s * kMmaStep),
                          vd + (((a * L::kVAtomBytes) >> 4) + s * kMmaStep), idesc_o, i != 0 ? 1u : (first_block ^ 1u));
      };
      auto wait_scores_operands = [&](int j) -> bool {
        return mbar_wait(&t.k_full_bar[j % kKvStages], (j / kKvStages) & 1, &abort_flag) &&
               mbar_wait(&t.s_empty_bar[j & 1], ((j >> 1) & 1) ^ 1, &abort_flag);
      };
      auto commit_scores = [&](int j) {
        umma_commit(&t.k_empty_bar[j % kKvStages]);
        umma_commit(&t.s_full_bar[j & 1]);
      };
      ok = mbar_wait(&t.q_full_bar, 0, &abort_flag);
      // The first two blocks' scores.
      for (int j = 0; j < 2 && j < num_blocks && ok; ++j) {
        ok = wait_scores_operands(j);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int i = 0; i < kScoreMmas; ++i) score_mma(tmem_base + (j & 1) * L::kSCols, (j & 1) ? kdesc_1 : kdesc_0, i);
        commit_scores(j);
      }
      for (int j = 0; j < num_blocks && ok; ++j) {
        const bool ahead = j + 2 < num_blocks;
        if (ahead && !wait_scores_operands(j + 2)) {
          ok = false;
          break;
        }
        if (!mbar_wait(&t.p_full_bar, j & 1, &abort_flag) ||
            !mbar_wait(&t.v_full_bar[j % kKvStages], (j / kKvStages) & 1, &abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // Two independent accumulator chains, issued in turn: an instruction into an accumulator
        // waits for the one before it, so in turn they take the time of one chain.
        static_assert(kScoreMmas == kOutMmas || kScoreMmas * 2 == kOutMmas, "interleave below");
        constexpr int kOutPerScore = kOutMmas / kScoreMmas;
        const bool odd = (j & 1) != 0;
        const uint32_t first_block = j == 0 ? 1u : 0u;
        const uint32_t s_tmem = tmem_base + (odd ? L::kSCols : 0);
        const uint64_t kd = odd ? kdesc_1 : kdesc_0, vd = odd ? vdesc_1 : vdesc_0, pd = odd ? pdesc_1 : pdesc0;
        if (ahead) {
#pragma unroll
          for (int i = 0; i < kScoreMmas; ++i) {
#pragma unroll
            for (int o = 0; o < kOutPerScore; ++o) out_mma(pd, vd, i * kOutPerScore + o, first_block);
            score_mma(s_tmem, kd, i);
          }
        } else {
#pragma unroll
          for (int i = 0; i < kOutMmas; ++i) out_mma(pd, vd, i, first_block);
        }
        umma_commit(&t.v_empty_bar[j % kKvStages]);
        umma_commit(&t.pv_done_bar[j & 1]);
        if (ahead) commit_scores(j + 2);
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusAttentionTimeout);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax and output
    // Two warps share 32 queries (warps w and w + 4 reach the same lanes of tensor memory): each
    // takes half of a block's keys, and half of the output's columns at the end.
    const uint32_t quarter = warp & 3;
    const uint32_t half = warp >> 2;
    constexpr int kMyKeys = kBlockKv / 2;  // = one swizzle atom of P
    static_assert(kMyKeys == kAtomElems, "a warp writes one atom of P");
    const int row = static_cast<int>(quarter) * 32 + static_cast<int>(lane);  // query within the CTA = lane of tensor memory
    const int q_pos = q0 + row + offset;  // this query's position among the keys
    const int key_first = first_key_of(p, q_pos), key_last = last_key_of(p, q_pos);  // what it sees
    // What every query of the CTA sees: a block of keys inside this range needs no masking.
    const int common_first = first_key_of(p, last_row + offset), common_last = last_key_of(p, q0 + offset);
    const uint32_t t_lane = tmem_base + ((quarter * 32u) << 16);
    // Where this row's 16-byte pieces go in an atom of P: piece c of row r sits at c ^ (r & 7).
    uint8_t *p_row = p_smem + half * L::kPAtomBytes + (row >> 3) * 1024 + (row & 7) * kAtomBytes;
    const uint32_t p_xor = static_cast<uint32_t>(row & 7);
    // The probabilities and the output in tensor memory are relative to m_used, which follows the
    // row's running maximum only when that has grown by more than kRescaleStep (in log2 units)
    // for some row of the warp: until then exp2(score - m_used) <= 2^kRescaleStep, which every
    // type here holds, and the output needs no rescaling. The normalisation at the end divides by
    // the sum taken relative to the same m_used, so the result is the same quotient. Both warps
    // of a pair see the same maxima, so they take the same decisions.
    constexpr float kRescaleStep = 8.0f;
    float m_used = -INFINITY;
    float l_run = 0.0f;  // this thread's half of the row's sum
    bool ok = true;
    uint32_t sc[kMyKeys / 32][32];  // this thread's scores of the block
    uint32_t v[32];
    // Waits, in order and each once, until `count` of the P V products have completed.
    int products_seen = 0;
    auto wait_products = [&](int count) -> bool {
      while (products_seen < count) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait(&t.pv_done_bar[products_seen & 1], (products_seen >> 1) & 1, &abort_flag));
        if (!ok) return false;
        ++products_seen;
      }
      tc_fence_after_sync();
      return true;
    };
    // Hands `mine` to the other warp of the pair and returns what that warp handed over; `n` counts
    // the exchanges (one mbarrier phase each).
    int exchanges = 0;
    auto exchange = [&](float mine, float *theirs) -> bool {
      t.pair_value[exchanges & 1][half][row] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&t.pair_bar[quarter]);
      ok = __all_sync(0xffffffffu, mbar_wait(&t.pair_bar[quarter], exchanges & 1, &abort_flag));
      if (!ok) return false;
      *theirs = t.pair_value[exchanges & 1][half ^ 1][row];
      ++exchanges;
      return true;
    };

    // This thread's scores of block j into registers in one round trip; the buffer goes back to
    // the MMAs at once.
    auto fetch_scores = [&](int j) -> bool {
      ok = __all_sync(0xffffffffu, mbar_wait(&t.s_full_bar[j & 1], (j >> 1) & 1, &abort_flag));
      if (!ok) return false;
      tc_fence_after_sync();
      const uint32_t t_s = t_lane + (j & 1) * L::kSCols + half * kMyKeys;
#pragma unroll
      for (int c = 0; c < kMyKeys / 32; ++c) tmem_ld_32x32(t_s + c * 32, sc[c]);
#pragma unroll
      for (int c = 0; c < kMyKeys / 32; ++c) tmem_ld_wait(sc[c]);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&t.s_empty_bar[j & 1]);
      return true;
    };

    fetch_scores(0);
    for (int j = 0; j < num_blocks && ok; ++j) {
      const int block_key0 = (block0 + j) * kBlockKv;
      const int key0 = block_key0 + static_cast<int>(half) * kMyKeys;  // this thread's first key
      // Does any key of this block need masking for any row of the CTA?
      const bool edge = block_key0 < common_first || block_key0 + kBlockKv - 1 > common_last;
      // Masked (edge blocks only), and the maximum over this thread's keys; the scale to log2
      // units is positive, so it is applied to the maximum here and to the scores inside the
      // exponent's multiply-add below.
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
      if (edge) {
#pragma unroll
        for (int c = 0; c < kMyKeys / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c * 32 + i;
            if (key > key_last || key < key_first) sc[c][i] = __float_as_uint(-INFINITY);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < kMyKeys / 32; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1]));
        }
      }
      float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      float m_other;
      if (!exchange(m_blk, &m_other)) break;
      m_blk = fmaxf(m_blk, m_other);
      // P V of block j - 2 is done: its P buffer, which this block takes, may be overwritten.
      if (!wait_products(j - 1)) break;
      if (__any_sync(0xffffffffu, m_blk > m_used + kRescaleStep)) {
        // The output is about to be rescaled: it has to be complete up to the previous block.
        if (!wait_products(j)) break;
        const float m_new = fmaxf(m_used, m_blk);
        const float alpha = exp2f(m_used - ((m_new == -INFINITY) ? 0.0f : m_new));  // 0 for a row's first keys
        l_run *= alpha;
        if (j > 0) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {  // this warp's half of the output's columns
            const uint32_t t_o = t_lane + L::kOCol + half * (D / 2) + c * 32;
            tmem_ld_32x32(t_o, v);
            tmem_ld_wait(v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(t_o, v);
          }
          tmem_st_wait();
        }
        m_used = m_new;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.0f : m_used;  // a row that has seen no key yet: every score is -inf
      // The probabilities, into shared memory as the A operand of P V.
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint8_t *atom = p_row + (j & 1) * L::kPBytes;
      // (One copy of the loop per 16-bit type, so that the choice is made once per block and not
      // once per pair of values.)
      auto emit = [&](auto bf16_tag) {
        constexpr int kBf16 = decltype(bf16_tag)::value ? 1 : 0;
#pragma unroll
        for (int c = 0; c < kMyKeys / 32; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(sc[c][i]), p.scale_log2, -m_sub));
            const float e1 = fast_exp2(fmaf(__uint_as_float(sc[c][i + 1]), p.scale_log2, -m_sub));
            sum4[(i >> 1) & 3] += e0 + e1;
            packed[i >> 1] = pack16(e0, e1, kBf16);
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t piece = static_cast<uint32_t>(c * 4 + g) ^ p_xor;
            *reinterpret_cast<uint4 *>(atom + piece * 16) =
                make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
          }
        }
      };
      if (p.is_bf16) {
        emit(std::true_type{});
      } else {
        emit(std::false_type{});
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // The next block's scores (ready since the product before last) are read before P is handed
      // over: the products that the hand-over starts would otherwise be under way when the read
      // is issued.
      if (j + 1 < num_blocks && !fetch_scores(j + 1)) break;
      fence_proxy_async_smem();  // the stores above, before the MMA's reads of them
      tc_fence_before_sync();    // and the rescaled output, before the MMA accumulates into it
      __syncwarp();
      if (lane == 0) mbar_arrive(&t.p_full_bar);
    }
    if (ok) wait_products(num_blocks);
    float l_other = 0.0f;
    if (ok) exchange(l_run, &l_other);
    if (ok) {
      const bool live = q0 + row < p.q_len;
      const float inv = 1.0f / (l_run + l_other);
      uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + batch * p.out_stride[0] + head * p.out_stride[1] +
                      static_cast<int64_t>(q0 + row) * p.out_stride[2] + half * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tmem_ld_32x32(t_lane + L::kOCol + half * (D / 2) + c * 32, v);
        tmem_ld_wait(v);
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack16(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv, p.is_bf16);
            w.y = pack16(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv, p.is_bf16);
            w.z = pack16(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv, p.is_bf16);
            w.w = pack16(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv, p.is_bf16);
            *reinterpret_cast<uint4 *>(dst + c * 32 + g * 8) = w;
          }
        }
      }
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, kStatusAttentionTimeout);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag != 0) {
    // A wait gave up: give copies that may still be in flight time to land before the shared
    // memory they target is released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, L::kTmemCols);
  }
}

// ---- two query tiles per CTA, probabilities in tensor memory -----------------------------------
//
// The kernel above reads both operands of both products from shared memory: 8 KB per instruction
// of 64 cycles is all the bandwidth shared memory has, and the probabilities written there and the
// K and V blocks arriving there take their share of it. Here a CTA owns two tiles of 128 queries of
// one head that walk the same keys, and a tile's probabilities never leave tensor memory: the
// softmax writes them (16-bit pairs, one row per lane) over the first half of the tile's own score
// buffer, and O += P V takes its A operand from there. Eight softmax warps (four per tile: a thread
// owns a whole row of a block's scores, so no two threads have to agree on a maximum), one producer
// warp, one issuing warp. The tiles share the K and V blocks (one ring of equal slots: K0 V0 K1 V1
// ...); tensor memory holds 2 x (128 + head_dim) <= 512 columns. Per tile the chain is serial
// (scores -> softmax -> P -> product -> the next scores, which overwrite P); the other tile's
// chain runs in its gaps.
constexpr int kTiles = 2;
constexpr int kTileWarps = 4;
constexpr int kSoftmaxWarps2 = kTiles * kTileWarps;
constexpr int kProducerWarp2 = kSoftmaxWarps2;
constexpr int kMmaWarp2 = kSoftmaxWarps2 + 1;
constexpr int kThreads2 = (kSoftmaxWarps2 + 2) * 32;
constexpr int kMaxSlots = 6;

struct Tail2 {
  uint64_t q_full_bar[kTiles];
  uint64_t slot_full_bar[kMaxSlots], slot_empty_bar[kMaxSlots];
  uint64_t s_full_bar[kTiles];   // MMA -> softmax: the tile's scores are in tensor memory
  uint64_t p_full_bar[kTiles];   // softmax -> MMA: the tile's probabilities are in tensor memory
  uint64_t pv_done_bar[kTiles];  // MMA -> softmax: the block is in the tile's output
  uint32_t tmem_base_slot;
  uint32_t abort_flag;
};

template <int D>
struct Layout2 {
  static constexpr int kQAtoms = D / kAtomElems;
  static constexpr int kQBytes = kQAtoms * kBlockQ * kAtomBytes;  // one tile's queries
  static constexpr int kSlotBytes = kQAtoms * kBlockKv * kAtomBytes;  // a block of K: 128 keys x head_dim
  static constexpr int kVAtoms = kBlockKv / kAtomElems;
  static constexpr int kVAtomBytes = D * kAtomBytes;
  static_assert(kVAtoms * kVAtomBytes == kSlotBytes, "a block of V^T fills a slot exactly as a block of K does");
  static constexpr int kRoom = (227 * 1024 - kTiles * kQBytes - static_cast<int>(sizeof(Tail2))) / kSlotBytes;
  static constexpr int kSlots = kRoom < kMaxSlots ? kRoom : kMaxSlots;
  static_assert(kSlots >= 3, "K of the next block, V of this one and a load in flight");
  static constexpr int kQOff = 0;
  static constexpr int kSlotOff = kQOff + kTiles * kQBytes;
  static constexpr int kTailOff = kSlotOff + kSlots * kSlotBytes;
  static constexpr int kSmemBytes = kTailOff + static_cast<int>(sizeof(Tail2));
  static constexpr int kSCols = kBlockKv;           // tile t's scores at column t * kSCols, its P over their first half
  static constexpr int kOCol = kTiles * kSCols;     // tile t's output at kOCol + t * D
  static constexpr int kTmemCols = 512;
  static_assert(kOCol + kTiles * D <= kTmemCols, "tensor memory holds 512 columns");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory");
};

template <int D>
__global__ void __launch_bounds__(kThreads2, 1)
attention2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_vt, const KernelParams p) {
  using L = Layout2<D>;
  constexpr int S = L::kSlots;
  extern __shared__ __align__(1024) uint8_t smem[];
  Tail2 &t = *reinterpret_cast<Tail2 *>(smem + L::kTailOff);
  volatile uint32_t &abort_flag = *reinterpret_cast<volatile uint32_t *>(&t.abort_flag);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0u, kStatusAttentionLayout);
    return;
  }
  // Under a causal mask the later queries have more keys to walk: those CTAs go first, so that the
  // grid's last round is made of short ones.
  const int q0 = static_cast<int>(p.mask_type != 0 ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * (kTiles * kBlockQ);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int offset = p.kv_len - p.q_len;
  // Both tiles walk the blocks of keys that some query of the CTA sees; a block none of a tile's
  // queries sees costs that tile a block of zero probabilities.
  const int last_row = min(q0 + kTiles * kBlockQ, p.q_len) - 1;
  const int kv_begin = first_key_of(p, q0 + offset);
  const int kv_end = last_key_of(p, last_row + offset) + 1;
  const int block0 = kv_begin / kBlockKv;
  const int num_blocks = (kv_end + kBlockKv - 1) / kBlockKv - block0;

  if (threadIdx.x == 0) {
    t.abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(&t.slot_full_bar[i], 1);
      mbar_init(&t.slot_empty_bar[i], 1);
    }
    for (int i = 0; i < kTiles; ++i) {
      mbar_init(&t.q_full_bar[i], 1);
      mbar_init(&t.s_full_bar[i], 1);
      mbar_init(&t.p_full_bar[i], kTileWarps);
      mbar_init(&t.pv_done_bar[i], 1);
    }
    fence_barrier_init();
  }
  if (warp == kProducerWarp2 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_vt);
  }
  if (warp == kMmaWarp2) {
    tmem_alloc<1>(&t.tmem_base_slot, L::kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = t.tmem_base_slot;

  auto q_tile = [&](int i) { return smem + L::kQOff + i * L::kQBytes; };
  auto slot = [&](int i) { return smem + L::kSlotOff + i * L::kSlotBytes; };

  // Load n of the ring (K of block n / 2 when n is even, V of it when odd) goes to slot n % S.
  if (warp == kProducerWarp2) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < kTiles; ++i) {
        mbar_arrive_expect_tx(&t.q_full_bar[i], L::kQBytes);
#pragma unroll
        for (int a = 0; a < L::kQAtoms; ++a) {
          tma_load_4d(q_tile(i) + a * kBlockQ * kAtomBytes, &tmap_q, &t.q_full_bar[i], a * kAtomBytes, q0 + i * kBlockQ, head,
                      batch);
        }
      }
      for (int n = 0; n < 2 * num_blocks && ok; ++n) {
        const int st = n % S, j = n >> 1;
        if (!mbar_wait(&t.slot_empty_bar[st], ((n / S) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&t.slot_full_bar[st], L::kSlotBytes);
        if ((n & 1) == 0) {
#pragma unroll
          for (int a = 0; a < L::kQAtoms; ++a) {
            tma_load_4d(slot(st) + a * kBlockKv * kAtomBytes, &tmap_k, &t.slot_full_bar[st], a * kAtomBytes,
                        (block0 + j) * kBlockKv, kv_head, batch);
          }
        } else if (p.v_direct) {  // v like k: 128 keys x 64 elements of head_dim per atom
#pragma unroll
          for (int a = 0; a < L::kQAtoms; ++a) {
            tma_load_4d(slot(st) + a * kBlockKv * kAtomBytes, &tmap_vt, &t.slot_full_bar[st], a * kAtomBytes,
                        (block0 + j) * kBlockKv, kv_head, batch);
          }
        } else {
#pragma unroll
          for (int a = 0; a < L::kVAtoms; ++a) {
            tma_load_3d(slot(st) + a * L::kVAtomBytes, &tmap_vt, &t.slot_full_bar[st],
                        ((block0 + j) * kBlockKv + a * kAtomElems) * 2, 0, batch * p.kv_heads + kv_head);
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusAttentionTimeout);
      }
    }
  } else if (warp == kMmaWarp2) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop and one lane issues: what an instruction takes (descriptors,
    // addresses) is then the same in every lane, which lets it live in uniform registers instead of
    // being moved there instruction by instruction by a lone thread.
    const bool issuer = lane == 0;
    {
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = umma_idesc(kBlockQ, kBlockKv, fmt, fmt);
      const uint32_t idesc_o = umma_idesc(kBlockQ, D, fmt, fmt);
      constexpr uint64_t kMmaStep = kMmaKBytes >> 4;
      constexpr int kMmasPerAtom = kAtomBytes / kMmaKBytes;
      constexpr int kScoreMmas = L::kQAtoms * kMmasPerAtom;
      constexpr int kOutMmas = L::kVAtoms * kMmasPerAtom;  // one per 16 keys: 8 columns of P each
      const uint64_t qdesc0 = umma_desc_sw128(smem_u32(q_tile(0)));
      const uint64_t sdesc0 = umma_desc_sw128(smem_u32(slot(0)));
      bool ok = true;
      auto scores = [&](int i, uint64_t kd) {  // S_i = Q_i K^T
        const uint32_t s_tmem = tmem_base + i * L::kSCols;
        const uint64_t qd = qdesc0 + static_cast<uint64_t>(i * (L::kQBytes >> 4));
#pragma unroll
        for (int m = 0; m < kScoreMmas; ++m) {
          const int a = m / kMmasPerAtom, s = m % kMmasPerAtom;
          if (issuer) umma_ss<kKindF16>(s_tmem, qd + (((a * kBlockQ * kAtomBytes) >> 4) + s * kMmaStep),
                            kd + (((a * kBlockKv * kAtomBytes) >> 4) + s * kMmaStep), idesc_s, m != 0 ? 1u : 0u);
        }
      };
      // With v as it lies, a slot's rows are keys: an instruction's 16 keys are 16 rows of 128 bytes
      // on, the operand is MN-major (bit 16 of the instruction descriptor) and its runs of 64
      // head_dim positions lie a 128-key atom apart.
      const uint32_t idesc_o_mn = idesc_o | (1u << 16);
      const uint64_t mn_fields = umma_desc_sw128_mn(0, kBlockKv * kAtomBytes) ^ umma_desc_sw128(0);
      auto product = [&](int i, uint64_t vd, uint32_t first_block) {  // O_i += P_i V
        const uint32_t o_tmem = tmem_base + L::kOCol + i * D;
        const uint32_t p_tmem = tmem_base + i * L::kSCols;
        if (p.v_direct) {
#pragma unroll
          for (int m = 0; m < kOutMmas; ++m) {
            if (issuer) umma_ts_f16(o_tmem, p_tmem + m * 8, (vd ^ mn_fields) + static_cast<uint64_t>(m * ((16 * kAtomBytes) >> 4)), idesc_o_mn,
                        m != 0 ? 1u : (first_block ^ 1u));
          }
        } else {
#pragma unroll
          for (int m = 0; m < kOutMmas; ++m) {
            const int a = m / kMmasPerAtom, s = m % kMmasPerAtom;
            if (issuer) umma_ts_f16(o_tmem, p_tmem + m * 8, vd + (((a * L::kVAtomBytes) >> 4) + s * kMmaStep), idesc_o,
                        m != 0 ? 1u : (first_block ^ 1u));
          }
        }
      };
      auto wait_full = [&](int n) -> bool { return mbar_wait(&t.slot_full_bar[n % S], (n / S) & 1, &abort_flag); };
      auto desc_of = [&](int n) -> uint64_t { return sdesc0 + static_cast<uint64_t>((n % S) * (L::kSlotBytes >> 4)); };
      for (int i = 0; i < kTiles && ok; ++i) ok = mbar_wait(&t.q_full_bar[i], 0, &abort_flag);
      if (ok && num_blocks > 0) ok = wait_full(0);
      if (ok && num_blocks > 0) {
        tc_fence_after_sync();
        for (int i = 0; i < kTiles; ++i) {
          scores(i, desc_of(0));
          if (issuer) umma_commit(&t.s_full_bar[i]);
        }
        if (issuer) umma_commit(&t.slot_empty_bar[0]);
      }
      for (int j = 0; j < num_blocks && ok; ++j) {
        const bool more = j + 1 < num_blocks;
        const int nv = 2 * j + 1, nk = 2 * j + 2;
        const uint32_t first_block = j == 0 ? 1u : 0u;
        for (int i = 0; i < kTiles && ok; ++i) {
          // (The second tile reads the slots the first one has just been seen to wait for.)
          if (!mbar_wait(&t.p_full_bar[i], j & 1, &abort_flag) || (i == 0 && (!wait_full(nv) || (more && !wait_full(nk))))) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          // The product reads P from the columns the next scores overwrite: the instructions of one
          // thread run in the order they were issued.
          product(i, desc_of(nv), first_block);
          if (!more && issuer) umma_commit(&t.pv_done_bar[i]);  // (a block's scores, which the softmax waits for, follow its product)
          if (more) {
            scores(i, desc_of(nk));
            if (issuer) umma_commit(&t.s_full_bar[i]);
          }
          if (i == kTiles - 1) {  // both tiles have read the two slots
            if (issuer) umma_commit(&t.slot_empty_bar[nv % S]);
            if (more && issuer) umma_commit(&t.slot_empty_bar[nk % S]);
          }
        }
      }
      if (!ok && issuer) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusAttentionTimeout);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax and output
    const int tile = static_cast<int>(warp >> 2);
    const uint32_t quarter = warp & 3;
    const int tq0 = q0 + tile * kBlockQ;  // the tile's first query
    const int row = static_cast<int>(quarter) * 32 + static_cast<int>(lane);
    const int q_pos = tq0 + row + offset;
    const int key_first = first_key_of(p, q_pos), key_last = last_key_of(p, q_pos);
    const int tile_last_row = min(tq0 + kBlockQ, p.q_len) - 1;
    // What every query of the tile sees (an empty range for a tile past the last query: every block
    // is then an edge block, and nothing of it is stored).
    const int common_first = first_key_of(p, tile_last_row + offset), common_last = last_key_of(p, tq0 + offset);
    const uint32_t t_lane = tmem_base + ((quarter * 32u) << 16);
    const uint32_t t_scores = t_lane + tile * L::kSCols;  // the row's 128 scores, then its 128 probabilities in 64 columns
    const uint32_t t_out = t_lane + L::kOCol + tile * D;
    constexpr int kChunks = kBlockKv / 32;
    static_assert(kChunks == 4, "four chunks of scores pack into the first two");
    constexpr float kRescaleStep = 8.0f;
    float m_used = -INFINITY;
    float l_run = 0.0f;
    bool ok = true;
    uint32_t sc[kChunks][32];

    for (int j = 0; j < num_blocks && ok; ++j) {
      // The row's scores of the block into registers in one round trip. (Scores of block j are
      // issued behind the product of block j - 1: once they are here the tile's output is complete
      // up to that block.)
      ok = __all_sync(0xffffffffu, mbar_wait(&t.s_full_bar[tile], j & 1, &abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < kChunks; ++c) tmem_ld_32x32(t_scores + c * 32, sc[c]);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) tmem_ld_wait(sc[c]);
      const int block_key0 = (block0 + j) * kBlockKv;
      const bool edge = block_key0 < common_first || block_key0 + kBlockKv - 1 > common_last;
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (edge) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = block_key0 + c * 32 + i;
            if (key > key_last || key < key_first) sc[c][i] = __float_as_uint(-INFINITY);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1]));
        }
      }
      const float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      if (__any_sync(0xffffffffu, m_blk > m_used + kRescaleStep)) {
        const float m_new = fmaxf(m_used, m_blk);
        const float alpha = exp2f(m_used - ((m_new == -INFINITY) ? 0.0f : m_new));
        l_run *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {  // sixteen columns at a time: the block's scores stay in registers
            uint32_t v[16];
            tmem_ld_32x16(t_out + c * 16, v);
            tmem_ld_wait(v);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x16(t_out + c * 16, v);
          }
        }
        m_used = m_new;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.0f : m_used;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      // The probabilities, packed in place: pair i of the row's keys becomes column i of its P
      // (a slot whose scores have been used by then).
      const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), neg_m2 = f2_pack(-m_sub, -m_sub);
      auto emit = [&](auto bf16_tag) {
        constexpr int kBf16 = decltype(bf16_tag)::value ? 1 : 0;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x = f2_fma(f2_pack(__uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1])), scale2, neg_m2);
            float e0, e1;
            if ((i & 6) != 6) {  // one pair in four goes through the cubic, the others through the special-function unit
              float x0, x1;
              f2_unpack(x, &x0, &x1);
              e0 = fast_exp2(x0);
              e1 = fast_exp2(x1);
            } else {
              exp2_pair_poly(x, &e0, &e1);
            }
            sum4[(i >> 1) & 3] += e0 + e1;
            sc[c >> 1][(c & 1) * 16 + (i >> 1)] = pack16(e0, e1, kBf16);
          }
        }
      };
      if (p.is_bf16) {
        emit(std::true_type{});
      } else {
        emit(std::false_type{});
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_st_32x32(t_scores, sc[0]);
      tmem_st_32x32(t_scores + 32, sc[1]);
      tmem_st_wait();          // the probabilities and a rescaled output are in tensor memory
      tc_fence_before_sync();  // before the MMAs that the hand-over starts
      __syncwarp();
      if (lane == 0) mbar_arrive(&t.p_full_bar[tile]);
    }
    // The last product.
    if (ok && num_blocks > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&t.pv_done_bar[tile], 0, &abort_flag));
      tc_fence_after_sync();
    }
    if (ok) {
      const bool live = tq0 + row < p.q_len;
      const float inv = 1.0f / l_run;
      uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + batch * p.out_stride[0] + head * p.out_stride[1] +
                      static_cast<int64_t>(tq0 + row) * p.out_stride[2];
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_out + c * 32, v);
        tmem_ld_wait(v);
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack16(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv, p.is_bf16);
            w.y = pack16(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv, p.is_bf16);
            w.z = pack16(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv, p.is_bf16);
            w.w = pack16(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv, p.is_bf16);
            *reinterpret_cast<uint4 *>(dst + c * 32 + g * 8) = w;
          }
        }
      }
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, kStatusAttentionTimeout);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == kMmaWarp2) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, L::kTmemCols);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      return reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// A byte tensor of `rank` dimensions, innermost contiguous, read in boxes of 128 bytes x box_rows
// rows of the second dimension, 128-byte swizzle, zeros outside.
bool make_tmap(CUtensorMap *map, const void *base, int rank, const uint64_t *dims, const uint64_t *strides_bytes,
               uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t d[4];
  cuuint64_t s[3];
  cuuint32_t box[4] = {static_cast<cuuint32_t>(kAtomBytes), box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) d[i] = dims[i];
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<cuuint32_t>(rank), const_cast<void *>(base), d, s, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int round_up(int x, int to) { return (x + to - 1) / to * to; }

template <int D>
cudaError_t launch(const AttentionArgs &a, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tvt,
                   const KernelParams &kp, const char **why) {
  using L = Layout<D>;
  auto kernel = attention_kernel<D>;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) {
      *why = "cudaFuncSetAttribute(max dynamic shared memory) failed";
      return e;
    }
    attr_set = true;
  }
  const dim3 grid(static_cast<unsigned>((a.q_len + kBlockQ - 1) / kBlockQ), static_cast<unsigned>(a.heads),
                  static_cast<unsigned>(a.batch));
  kernel<<<grid, kThreads, L::kSmemBytes, a.stream>>>(tq, tk, tvt, kp);
  return cudaGetLastError();
}

template <int D>
cudaError_t launch2(const AttentionArgs &a, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tvt,
                    const KernelParams &kp, const char **why) {
  using L = Layout2<D>;
  auto kernel = attention2_kernel<D>;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) {
      *why = "cudaFuncSetAttribute(max dynamic shared memory) failed";
      return e;
    }
    attr_set = true;
  }
  const int per_cta = kTiles * kBlockQ;
  const dim3 grid(static_cast<unsigned>((a.q_len + per_cta - 1) / per_cta), static_cast<unsigned>(a.heads),
                  static_cast<unsigned>(a.batch));
  kernel<<<grid, kThreads2, L::kSmemBytes, a.stream>>>(tq, tk, tvt, kp);
  return cudaGetLastError();
}

}  // namespace

bool attention_supported(const AttentionArgs &a, const char **why) {
  auto fail = [&](const char *m) {
    *why = m;
    return false;
  };
  if (a.head_dim != 64 && a.head_dim != 128) return fail("head_dim is not 64 or 128");
  if (a.batch < 0 || a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads != 0) return fail("heads is not a multiple of kv_heads");
  if (a.batch > 65535 || a.heads > 65535) return fail("more than 65535 heads or batches");
  if (a.q_len < 0 || a.kv_len <= 0) return fail("no keys");
  if (a.mask_type < 0 || a.mask_type > 3) return fail("unknown mask");
  if ((a.mask_type == 1 || a.mask_type == 2) && a.kv_len < a.q_len) return fail("the causal masks need at least as many keys as queries");
  if (a.mask_type == 3 && a.kv_len != a.q_len) return fail("the block diagonal mask is self-attention: as many keys as queries");
  if ((a.mask_type >= 2) != (a.block_size > 0)) return fail("a block size goes with a block mask, and only with one");
  const void *ptrs[4] = {a.q, a.k, a.v, a.out};
  for (const void *ptr : ptrs) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail("an operand does not start on a 16-byte boundary");
  }
  const int64_t *strides[4] = {a.q_stride, a.k_stride, a.v_stride, a.out_stride};
  for (const int64_t *s : strides) {
    for (int i = 0; i < 3; ++i) {
      if (s[i] < 0 || s[i] % 8 != 0) return fail("a stride is negative or not a multiple of 8 elements");
    }
  }
  // q, k and out are read and written through tensor maps, which cannot repeat a dimension: a
  // stride of 0 (a broadcast view) over an extent above 1 is refused here rather than read at the
  // wrong addresses. Only a dimension of extent 1, whose stride indexes nothing, may carry one.
  // (v is gathered by the transposing kernel with its true strides and may repeat.)
  const int q_extent[3] = {a.batch, a.heads, a.q_len};
  const int k_extent[3] = {a.batch, a.kv_heads, a.kv_len};
  for (int i = 0; i < 3; ++i) {
    if ((q_extent[i] > 1 && (a.q_stride[i] == 0 || a.out_stride[i] == 0)) || (k_extent[i] > 1 && a.k_stride[i] == 0)) {
      return fail("q, k or out repeats a dimension through a stride of 0 (a broadcast view)");
    }
  }
  return true;
}

size_t attention_scratch_bytes(int batch, int kv_heads, int kv_len, int head_dim) {
  return static_cast<size_t>(batch) * kv_heads * head_dim * round_up(kv_len, kPadKv) * 2;
}

AttentionPlan attention_plan(const AttentionArgs &a) {
  // Two tiles of queries per CTA where a head has more than one tile of them; the block diagonal
  // mask, whose tiles see different keys, and short query runs keep one tile per CTA.
  static const bool one_tile_only = [] {
    const char *e = std::getenv("FLINT_SM100_ATTENTION_ONE_TILE");
    return e && e[0] == '1';
  }();
  static const bool transposed_v_only = [] {
    const char *e = std::getenv("FLINT_SM100_ATTENTION_TRANSPOSED_V");
    return e && e[0] == '1';
  }();
  const bool block_diagonal = a.mask_type == 3 && a.block_size < a.kv_len;  // (one block over every key is no mask)
  AttentionPlan plan;
  plan.two_tiles = a.q_len > kBlockQ && !block_diagonal && !one_tile_only;
  // The two-tile kernel reads v as it lies (a tensor map like k's, the operand MN-major) unless v
  // repeats a dimension through a stride of 0, which only the transposing kernel can follow.
  const int v_extent[3] = {a.batch, a.kv_heads, a.kv_len};
  bool v_plain = true;
  for (int i = 0; i < 3; ++i) v_plain = v_plain && !(v_extent[i] > 1 && a.v_stride[i] == 0);
  plan.v_direct = plan.two_tiles && v_plain && !transposed_v_only;
  plan.launches = plan.v_direct ? 1 : 2;
  return plan;
}

cudaError_t attention(const AttentionArgs &a, const char **why) {
  *why = "";
  if (!attention_supported(a, why)) return cudaErrorInvalidValue;
  if (a.batch == 0 || a.q_len == 0) return cudaSuccess;
  const int d = a.head_dim;
  const int kv_pad = round_up(a.kv_len, kPadKv);

  KernelParams kp = {};
  kp.out = a.out;
  for (int i = 0; i < 3; ++i) kp.out_stride[i] = a.out_stride[i];
  kp.is_bf16 = a.is_bf16;
  kp.heads = a.heads;
  kp.kv_heads = a.kv_heads;
  kp.group = a.heads / a.kv_heads;
  kp.q_len = a.q_len;
  kp.kv_len = a.kv_len;
  kp.mask_type = a.mask_type;
  kp.block_size = a.block_size;
  if (a.mask_type >= 2 && a.block_size >= a.kv_len) {  // one block holds every key: no mask at all
    kp.mask_type = 0;
    kp.block_size = 0;
  }
  kp.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(d));
  kp.status = a.status;
  const AttentionPlan plan = attention_plan(a);
  const bool two_tiles = plan.two_tiles;
  kp.v_direct = plan.v_direct ? 1 : 0;

  if (!kp.v_direct) {
    const dim3 tgrid(static_cast<unsigned>(kv_pad / 64), static_cast<unsigned>(d / 64),
                     static_cast<unsigned>(a.batch * a.kv_heads));
    transpose_v_kernel<<<tgrid, 256, 0, a.stream>>>(reinterpret_cast<const uint16_t *>(a.v), a.v_stride[0], a.v_stride[1],
                                                    a.v_stride[2], a.kv_heads, a.kv_len, kv_pad, d,
                                                    reinterpret_cast<uint16_t *>(a.v_transposed));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      *why = "launching the transposition of v";
      return e;
    }
  }

  // q, k (and v as it lies) as (head_dim bytes, positions, heads, batch); a size-1 dimension's
  // stride is never used but has to pass the encoder's checks.
  auto dims4 = [&](int len, int heads, uint64_t *dims) {
    dims[0] = static_cast<uint64_t>(d) * 2;
    dims[1] = static_cast<uint64_t>(len);
    dims[2] = static_cast<uint64_t>(heads);
    dims[3] = static_cast<uint64_t>(a.batch);
  };
  auto strides4 = [&](const int64_t *s, uint64_t *out) {
    out[0] = static_cast<uint64_t>(s[2] > 0 ? s[2] : d) * 2;
    out[1] = static_cast<uint64_t>(s[1] > 0 ? s[1] : d) * 2;
    out[2] = static_cast<uint64_t>(s[0] > 0 ? s[0] : d) * 2;
  };
  uint64_t dims[4], strides[3];
  CUtensorMap tq, tk, tvt;
  dims4(a.q_len, a.heads, dims);
  strides4(a.q_stride, strides);
  if (!make_tmap(&tq, a.q, 4, dims, strides, kBlockQ)) {
    *why = "cuTensorMapEncodeTiled refused q";
    return cudaErrorInvalidValue;
  }
  dims4(a.kv_len, a.kv_heads, dims);
  strides4(a.k_stride, strides);
  if (!make_tmap(&tk, a.k, 4, dims, strides, kBlockKv)) {
    *why = "cuTensorMapEncodeTiled refused k";
    return cudaErrorInvalidValue;
  }
  if (kp.v_direct) {
    strides4(a.v_stride, strides);
    if (!make_tmap(&tvt, a.v, 4, dims, strides, kBlockKv)) {
      *why = "cuTensorMapEncodeTiled refused v";
      return cudaErrorInvalidValue;
    }
  } else {
    uint64_t vdims[3] = {static_cast<uint64_t>(kv_pad) * 2, static_cast<uint64_t>(d),
                         static_cast<uint64_t>(a.batch) * a.kv_heads};
    uint64_t vstrides[2] = {static_cast<uint64_t>(kv_pad) * 2, static_cast<uint64_t>(d) * kv_pad * 2};
    if (!make_tmap(&tvt, a.v_transposed, 3, vdims, vstrides, static_cast<uint32_t>(d))) {
      *why = "cuTensorMapEncodeTiled refused the transposed v";
      return cudaErrorInvalidValue;
    }
  }
  if (two_tiles) return d == 64 ? launch2<64>(a, tq, tk, tvt, kp, why) : launch2<128>(a, tq, tk, tvt, kp, why);
  if (d == 64) return launch<64>(a, tq, tk, tvt, kp, why);
  return launch<128>(a, tq, tk, tvt, kp, why);
}

}  // namespace flsm100
