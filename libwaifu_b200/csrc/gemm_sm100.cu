// The sm_100a GEMM kernels behind flint's quantized matmul (replaces the CUTLASS 2.x Sm80
// mma.sync kernel of flint/cuda/gemm_fp8_cutlass.cu:94-197,267-305).
//
// One persistent CTA per SM (or one pair of CTAs per two SMs), twelve warps:
//   warps 0-7  epilogue: tensor memory -> registers -> scale/bias/GELU/residual -> 16-bit results,
//              which leave through a per-warp shared-memory buffer and TMA stores. Warp w reads
//              the 32 accumulator rows of lane quarter (w & 3) and the column half (w >> 2) of the tile.
//   warp  8    producer: TMA tile loads of A and B (and the NVFP4 scale-factor tiles) into a
//              ring of shared-memory stages, signalled through mbarriers
//   warp  9    MMA: one thread issues tcgen05.mma on the staged tiles, accumulating in tensor
//              memory; tcgen05.commit hands stages back to the producer and finished
//              accumulators to the epilogue
//   warps 10-11 in the NVFP4 kind one thread of them copies scale factors into tensor memory; in
//              the scatter form (a product gathered on several GPUs) the epilogue's TMA stores go
//              to every destination matrix, this GPU's and its peers', and these warps are idle;
//              only where a destination cannot be described by a tensor map do they push: once the
//              epilogue has written a tile into this GPU's matrix they copy its rows to the peers'
//              matrices, 512 contiguous bytes per store instruction, over NVLink.
// The mixed form (a half activation against an e4m3 weight that is NOT narrowed, flint's
// fl_fp8_matmul) divides the twelve differently: warps 0-3 epilogue (a warp takes its 32 rows of
// all the tile's columns), warp 4 producer, warp 5 MMA, warps 6-11 converters. The weight tile
// arrives as e4m3 bytes and the converters widen it exactly to half into the swizzled 16-bit tile
// the UMMA reads, so the weight crosses HBM and L2 once, as bytes (the reference widens in
// registers inside its main loop, flint/cuda/gemm_fp8_cutlass.cu:142-149). Six warps because the
// conversion instruction's units are per scheduler and two warps could not keep up with the UMMAs.
// The accumulator is double-buffered in tensor memory so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Schedule. Tiles are handed out round by round, one per unit (a CTA or a CTA pair). When the
// tile count is not a multiple of the unit count the last round would run nearly empty (816 pair
// tiles on 74 pairs: eleven full rounds and one of two tiles), so, given a workspace, the last
// full round and the remainder are pooled and their K stages dealt out evenly instead ("stream-K"
// over the last one-and-a-bit rounds): every unit gets a contiguous run of stages of that pool,
// which is the end of one tile, possibly whole tiles, and the beginning of another. A tile that is
// cut this way has exactly two holders (a run is at least one tile long). A holder's epilogue
// warps look at a per-tile, per-warp counter: if the other holder has not counted itself in yet,
// they write their part of the fp32 accumulator to the workspace and count themselves in; if it
// has, they add its part to their accumulator (head + tail, the same sum whoever comes second)
// and run the ordinary epilogue on it. A unit computes its head piece first and its tail piece
// last, so the write happens early, under the main loops that follow, and the end of the kernel
// only has the read. Nobody waits for anybody: there is no spin on another unit's progress.
//
// Every operand row in a stage is 128 bytes (64 half / 128 e4m3 / 256 e2m1 elements) in the
// 128-byte swizzle, and one tcgen05.mma consumes 32 bytes of K from every row, so the three
// element kinds share all of the addressing and differ only in the instruction issued.
#include "gemm_sm100.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kBlockM = 128;
constexpr int kRowBytes = 128;          // bytes of K per operand row per stage
constexpr int kMmaKBytes = 32;          // bytes of K one tcgen05.mma consumes per row
constexpr int kMmasPerStage = kRowBytes / kMmaKBytes;
constexpr int kSfTileBytes = 512;       // 128 rows x 4 scale factors
constexpr int kNumWarps = 12;
constexpr int kNumThreads = kNumWarps * 32;
constexpr int kMaxEpilogueWarps = 8;
constexpr int kPusherWarps = 2;
// Who does what among the twelve warps. Tensor memory lets a warp read the 32 lanes of its index
// modulo 4 only, so epilogue warps come in fours, each four covering a tile's 128 rows and one
// share of its columns. The mixed form gives up one of the two fours to have six converter warps:
// widening is conversion-instruction bound, and those units are per scheduler.
template <bool B8>
struct Roles {
  static constexpr int kEpilogueWarps = B8 ? 4 : 8;
  static constexpr int kColumnShares = kEpilogueWarps / 4;
  static constexpr int kProducerWarp = kEpilogueWarps;
  static constexpr int kMmaWarp = kEpilogueWarps + 1;
  static constexpr int kAuxWarp0 = kEpilogueWarps + 2;       // pushers / scale-factor copier, or converters
  static constexpr int kAuxWarps = kNumWarps - kAuxWarp0;    // 2, or 6
};
// Tiles are walked in bands of tile columns, columns fastest inside a band, so that the tiles in
// flight at one time share a compact set of A and B rows in L2. A matrix up to kBandMax tile
// columns wide is one band (every A row block is then fetched from HBM once); wider ones are cut
// into bands of kBandTiles.
constexpr int kStreamKMinSavedStages = 40;
constexpr int kBandTiles = 8;
constexpr int kBandMax = 16;

// One map per destination of the staged epilogue.
struct OutMaps {
  CUtensorMap at[kMaxGemmOutputs];
};

struct KernelParams {
  int m, n;
  int num_kb;  // stages of K per tile
  int tiles_m, tiles_n;
  const uint8_t *sfa;
  const uint8_t *sfb;
  int sf_k_tiles;
  const float *row_scale;
  const float *col_scale;
  int col_scale_scalar;
  const float *global_scale;
  const void *bias;
  const void *residual;
  int residual_rows;
  int rows_per_group;
  long long residual_ld;
  int act;
  float *row_amax;  // (m) or null: per-row maximum of the rounded results' magnitudes, by atomicMax on the float's bits
  int out_bf16;
  void *out[kMaxGemmOutputs];  // destinations of every tile: one, or this GPU's and its peers' copies
  int num_out;
  long long out_ld;            // pitch of the destination matrices in elements
  int out_col0;                // first destination column of this product
  int out_vector;  // the outputs' bases are 16-byte aligned: 16-byte stores; else 2-byte stores
  int out_staged;  // results leave through shared memory and TMA stores (tmap_out), residual rows come in coalesced
  uint32_t *status;
  // Schedule: `dp_rounds` rounds of whole tiles (tile = round * units + unit), then `sk_tiles`
  // tiles from `sk_first_tile` on whose K stages are dealt out evenly over the units (0: none).
  int dp_rounds;
  int sk_tiles;
  int sk_first_tile;
  float *sk_partials;     // units * 2 slots of one tile's fp32 accumulator each (per CTA: 128 x BLOCK_N)
  uint32_t *sk_counters;  // sk_tiles * CTAS * 8 counters, zero between launches
};

// One piece of work of a unit: the K stages [kb0, kb1) of a tile.
struct WorkItem {
  int tile;
  int kb0, kb1;
  int sk_tile;   // index among the stream-K tiles (counters), -1 for a whole tile of the data-parallel rounds
  bool partial;  // part of a tile: the accumulator goes to the workspace
  bool head;     // partial only: this is the tile's first part (else its last)
};

// The sequence of a unit's work items; every role of a CTA walks the same sequence: the rounds of
// whole tiles, then the unit's run [sk_begin, sk_end) of the stream-K pool in this order: the
// beginning of the tile the run ends in (a head), the whole tiles inside the run, the end of the
// tile the run starts in (a tail). That order makes every cut tile's head the first thing its
// holder does in this part and its tail the last thing the other holder does: the head's
// accumulator goes to the workspace early, under the main loops that follow, and at the end of the
// kernel a unit only reads one finished part back.
struct WorkWalk {
  int unit, num_units, num_tiles, num_kb, dp_rounds, sk_first_tile;
  long long sk_begin, sk_end;
  int round;
  int phase;       // of the stream-K part: 0 head, 1 whole tiles, 2 tail, 3 done
  int whole_tile;  // next whole tile of the run (index within the stream-K tiles)

  __device__ __forceinline__ WorkWalk(const KernelParams &p, int unit_, int num_units_)
      : unit(unit_), num_units(num_units_), num_tiles(p.tiles_m * p.tiles_n), num_kb(p.num_kb), dp_rounds(p.dp_rounds),
        sk_first_tile(p.sk_first_tile), round(0), phase(p.sk_tiles > 0 ? 0 : 3) {
    const long long total = static_cast<long long>(p.sk_tiles) * p.num_kb;
    sk_begin = total * unit_ / num_units_;
    sk_end = total * (unit_ + 1) / num_units_;
    whole_tile = static_cast<int>((sk_begin + num_kb - 1) / num_kb);
  }

  __device__ __forceinline__ bool next(WorkItem *it) {
    if (round < dp_rounds) {
      const int tile = round * num_units + unit;
      ++round;
      if (tile >= num_tiles) return false;  // only in the last round of a schedule without a stream-K part
      *it = WorkItem{tile, 0, num_kb, -1, false, false};
      return true;
    }
    if (phase == 0) {
      phase = 1;
      const int t = static_cast<int>(sk_end / num_kb);
      const int len = static_cast<int>(sk_end - static_cast<long long>(t) * num_kb);
      if (len > 0) {  // the run ends inside tile t: its first `len` stages
        *it = WorkItem{sk_first_tile + t, 0, len, t, true, true};
        return true;
      }
    }
    if (phase == 1) {
      if (static_cast<long long>(whole_tile + 1) * num_kb <= sk_end) {
        *it = WorkItem{sk_first_tile + whole_tile, 0, num_kb, whole_tile, false, false};
        ++whole_tile;
        return true;
      }
      phase = 2;
    }
    if (phase == 2) {
      phase = 3;
      const int t = static_cast<int>(sk_begin / num_kb);
      const int kb0 = static_cast<int>(sk_begin - static_cast<long long>(t) * num_kb);
      if (kb0 > 0) {  // the run starts inside tile t: its stages from kb0 on
        *it = WorkItem{sk_first_tile + t, kb0, num_kb, t, true, false};
        return true;
      }
    }
    return false;
  }
};

// CTAS == 2: a pair of CTAs (one cluster) shares a 256 x BLOCK_N tile through cta_group::2 UMMAs;
// each CTA stages its own 128 rows of A and its own half of the BLOCK_N rows of B.
template <int BLOCK_N, bool NVF4, int CTAS = 1, bool B8 = false>
struct Config : Roles<B8> {
  using Roles<B8>::kEpilogueWarps;
  using Roles<B8>::kColumnShares;
  static_assert(!(NVF4 && B8), "the mixed form is a 16-bit kind");
  static_assert(BLOCK_N % 64 == 0, "each epilogue warp takes whole 32-column chunks of its share of a tile");
  static constexpr int kABytes = kBlockM * kRowBytes;
  static constexpr int kBRows = BLOCK_N / CTAS;
  static constexpr int kBBytes = kBRows * kRowBytes;
  // Scale factors: A has one 128-row group; B is loaded as whole 128-row groups that cover the
  // tile (a 192-wide tile starts mid-group on odd tiles, so it needs two).
  static constexpr int kSfbGroups = NVF4 ? (BLOCK_N + 127) / 128 : 0;
  static constexpr int kSfaBytes = NVF4 ? kMmasPerStage * kSfTileBytes : 0;
  static constexpr int kSfbBytes = NVF4 ? kSfbGroups * kMmasPerStage * kSfTileBytes : 0;
  // Mixed form: 64 raw e4m3 bytes per B row per stage (the 64 K positions a 16-bit stage holds).
  static constexpr int kRawRowBytes = 64;
  static constexpr int kRawBytes = B8 ? kBRows * kRawRowBytes : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes + kRawBytes;
  // Each epilogue warp keeps its own copy of its columns' scale and bias as fp32 (a private copy
  // needs no barrier between warps, so no wait in the epilogue is unbounded).
  static constexpr int kHalfN = BLOCK_N / kColumnShares;  // columns of a tile one epilogue warp handles
  static constexpr int kColParamBytes = kEpilogueWarps * 2 * kHalfN * 4;
  // Each epilogue warp also has 32 rows x 64 bytes of its own (one 32-column chunk of 16-bit
  // results in the 64-byte swizzle) through which results leave by TMA store and residual rows
  // arrive by coalesced loads: a lane owns a row of the accumulator, and 16-byte accesses to 32
  // different rows of global memory per instruction are what bounded the epilogue before.
  static constexpr int kOutStageBytesPerWarp = 32 * 64;
  static constexpr int kOutStageBytes = kEpilogueWarps * kOutStageBytesPerWarp;
  static constexpr int kSmemBudget = 227 * 1024 - 2048 - kColParamBytes - kOutStageBytes;
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kOutStageOffset = kStages * kStageBytes;  // 1024-byte aligned (stage sizes are)
  static constexpr int kColParamOffset = kOutStageOffset + kOutStageBytes;
  static constexpr int kSmemBytes = kColParamOffset + kColParamBytes + 1024;  // + slack to align to 1024
  static_assert(kStageBytes % 512 == 0, "the output staging behind the stages has to stay 512-byte aligned");
  // Tensor memory columns: two accumulators, then two sets of one stage's scale factors. The
  // copies into a set are issued by a thread of their own, a stage ahead of the MMAs that read
  // the other set: issued by the MMA thread itself they execute in order with its MMAs, and
  // cost as much as those.
  static constexpr int kAccCols = 2 * BLOCK_N;
  static constexpr int kSfaCols = NVF4 ? kMmasPerStage * 4 : 0;
  static constexpr int kSfbColsPerMma = NVF4 ? kSfbGroups * 4 : 0;
  static constexpr int kSfbCols = kMmasPerStage * kSfbColsPerMma;
  static constexpr int kSfSetCols = kSfaCols + kSfbCols;
  static constexpr int kUsedCols = kAccCols + 2 * kSfSetCols;
  static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                   : kUsedCols <= 256 ? 256 : 512;
  static_assert(kUsedCols <= 512, "tensor memory holds 512 columns");
  static_assert(kStages >= 2, "need at least two stages");
};

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) == x * sigmoid(2u) == x / (1 + 2^z), u = sqrt(2/pi) (x + 0.044715 x^3),
  // z = -2 u log2(e) = x (c0 + c1 x^2)
  // (waifu/src/krea2/dit.rs:170-188 spells the same function as seven graph nodes).
  // Five FP32 operations and two special-function operations; both approximations are good to
  // about 2^-22, far inside the 16-bit output step. x -> -inf gives 2^z = inf, 1/inf = 0, -0.
  constexpr float kC0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  constexpr float kC1 = kC0 * 0.044715f;
  const float z = x * fmaf(x * x, kC1, kC0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  return x * r;
}

__device__ __forceinline__ float load16(const void *p, long long idx, int is_bf16) {
  if (is_bf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[idx]);
  return __half2float(reinterpret_cast<const __half *>(p)[idx]);
}

__device__ __forceinline__ uint32_t pack16(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Tile index -> (row tile, column tile).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int *tm, int *tn) {
  const int band_tiles = tiles_n <= kBandMax ? tiles_n : kBandTiles;
  const int per_band = band_tiles * tiles_m;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int width = min(band_tiles, tiles_n - band * band_tiles);
  *tm = r / width;
  *tn = band * band_tiles + (r - (*tm) * width);
}

template <int KIND, int BLOCK_N, int CTAS, bool B8>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
               const __grid_constant__ OutMaps tmaps_out, const KernelParams p) {
  constexpr bool NVF4 = (KIND == kKindNvf4);
  using Cfg = Config<BLOCK_N, NVF4, CTAS, B8>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int kEpilogueWarps = Cfg::kEpilogueWarps;
  constexpr int kProducerWarp = Cfg::kProducerWarp;
  constexpr int kMmaWarp = Cfg::kMmaWarp;
  constexpr int kPusherWarp0 = Cfg::kAuxWarp0;
  constexpr int kConverterWarps = Cfg::kAuxWarps;
  // A work unit is one CTA, or one pair of CTAs; rank 0 of a pair is its leader: it owns the
  // barriers both producers signal and it alone issues the UMMAs.
  const uint32_t cta_rank = (CTAS == 2) ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = blockIdx.x / CTAS;
  const int num_units = gridDim.x / CTAS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ __align__(8) uint64_t tile_done_bar[2];  // epilogue -> pushers: the tile is in this GPU's matrix
  __shared__ __align__(8) uint64_t sf_full_bar[2];    // NVFP4: a set of scale factors is in tensor memory
  __shared__ __align__(8) uint64_t sf_empty_bar[2];   // NVFP4: the MMAs that read the set are done
  __shared__ __align__(8) uint64_t raw_full_bar[B8 ? STAGES : 1];  // mixed form: a stage's e4m3 weight bytes have landed
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile uint32_t abort_flag;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  // Several destinations (a product gathered on several GPUs): in the staged form every chunk leaves
  // shared memory once per destination by TMA; otherwise the pusher warps copy this GPU's finished
  // tile to the others.
  const bool scatter = p.num_out > 1 && !p.out_staged;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      // Mixed form: a stage is full when the A bytes have landed (the producer's arrival with
      // its byte count) and every converter warp of the unit has written its share of B.
      mbar_init(&full_bar[s], B8 ? 1 + kConverterWarps * CTAS : 1);
      mbar_init(&empty_bar[s], 1);
      if constexpr (B8) mbar_init(&raw_full_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      // In a pair both CTAs' epilogues report to the leader. In the scatter form the pushers hold
      // the accumulator too, which keeps the epilogue from running two tiles ahead of them.
      mbar_init(&acc_empty_bar[s], (kEpilogueWarps + (scatter ? kPusherWarps : 0)) * CTAS);
      mbar_init(&tile_done_bar[s], kEpilogueWarps);
      mbar_init(&sf_full_bar[s], 1);
      mbar_init(&sf_empty_bar[s], 1);
    }
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.out_staged) {
      for (int d = 0; d < p.num_out; ++d) tma_prefetch_desc(&tmaps_out.at[d]);
    }
  }
  if (warp == kMmaWarp) {
    tmem_alloc<CTAS>(&tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the other CTA's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  // Everything above touched no global memory, so it may overlap the tail of the kernel before
  // this one in the stream (the activation quantiser); from here on its results are needed.
  griddep_wait();
  griddep_launch_dependents();

  auto stage_a = [&](int s) { return smem + s * Cfg::kStageBytes; };
  auto stage_b = [&](int s) { return smem + s * Cfg::kStageBytes + Cfg::kABytes; };
  auto stage_sfa = [&](int s) { return smem + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes; };
  auto stage_sfb = [&](int s) { return smem + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes + Cfg::kSfaBytes; };
  auto stage_raw = [&](int s) { return smem + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes; };
  (void)stage_raw;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkWalk walk(p, unit, num_units);
      WorkItem item;
      while (ok && walk.next(&item)) {
        int tm, tn;
        tile_coords(item.tile, p.tiles_m, p.tiles_n, &tm, &tn);
        const int m0 = tm * (kBlockM * CTAS) + static_cast<int>(cta_rank) * kBlockM;
        const int n0 = tn * BLOCK_N;
        for (int kb = item.kb0; kb < item.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag)) {
            ok = false;
            break;
          }
          // Scale-factor tiles of this k block (NVFP4): kMmasPerStage consecutive 512-byte tiles
          // per 128-row group, addressed as rows of a (groups * sf_k_tiles, 512 byte) matrix. A
          // CTA loads the group of its own A rows and every group its tile's B columns touch (in
          // a pair both CTAs need all of B's factors, since each multiplies its rows by all
          // BLOCK_N columns).
          const int sfa_row = (tm * CTAS + static_cast<int>(cta_rank)) * p.sf_k_tiles + kb * kMmasPerStage;
          const int sfb_row0 = (n0 / 128) * p.sf_k_tiles + kb * kMmasPerStage;
          if constexpr (B8) {
            // The weight's bytes go to the raw part of the stage under a barrier of this CTA's own,
            // which its converter warps wait on; only A counts on the stage's barrier.
            mbar_arrive_expect_tx(&raw_full_bar[stage], Cfg::kRawBytes);
            tma_load_2d(stage_raw(stage), &tmap_b, &raw_full_bar[stage], kb * Cfg::kRawRowBytes,
                        n0 + static_cast<int>(cta_rank) * Cfg::kBRows);
            if constexpr (CTAS == 2) {
              if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kABytes);
              tma_load_2d_pair(stage_a(stage), &tmap_a, map_to_cta(smem_u32(&full_bar[stage]), 0), kb * kRowBytes, m0);
            } else {
              mbar_arrive_expect_tx(&full_bar[stage], Cfg::kABytes);
              tma_load_2d(stage_a(stage), &tmap_a, &full_bar[stage], kb * kRowBytes, m0);
            }
          } else if constexpr (CTAS == 2) {
            // Both CTAs' bytes are counted on the leader's barrier, which the leader arms.
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            tma_load_2d_pair(stage_a(stage), &tmap_a, bar, kb * kRowBytes, m0);
            tma_load_2d_pair(stage_b(stage), &tmap_b, bar, kb * kRowBytes,
                             n0 + static_cast<int>(cta_rank) * Cfg::kBRows);
            if constexpr (NVF4) {
              tma_load_2d_pair(stage_sfa(stage), &tmap_sfa, bar, 0, sfa_row);
#pragma unroll
              for (int g = 0; g < Cfg::kSfbGroups; ++g) {
                tma_load_2d_pair(stage_sfb(stage) + g * kMmasPerStage * kSfTileBytes, &tmap_sfb, bar, 0,
                                 sfb_row0 + g * p.sf_k_tiles);
              }
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            tma_load_2d(stage_a(stage), &tmap_a, &full_bar[stage], kb * kRowBytes, m0);
            tma_load_2d(stage_b(stage), &tmap_b, &full_bar[stage], kb * kRowBytes, n0);
            if constexpr (NVF4) {
              tma_load_2d(stage_sfa(stage), &tmap_sfa, &full_bar[stage], 0, sfa_row);
#pragma unroll
              for (int g = 0; g < Cfg::kSfbGroups; ++g) {
                tma_load_2d(stage_sfb(stage) + g * kMmasPerStage * kSfTileBytes, &tmap_sfb, &full_bar[stage], 0,
                            sfb_row0 + g * p.sf_k_tiles);
              }
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusProducerTimeout));
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issue
    // The whole warp of the leader walks the loop and one lane issues: what an instruction takes is
    // then the same in every lane.
    if (leader) {
      const bool issuer = lane == 0;
      // e4m3 is format 0 of kind::f8f6f4; fp16 / bf16 are formats 0 / 1 of kind::f16.
      // (The mixed form exists for half only: both operands of a UMMA share one 16-bit format.)
      constexpr uint32_t kFmt = (KIND == kKindBF16) ? 1u : 0u;
      constexpr uint32_t idesc =
          NVF4 ? umma_idesc_nvf4(kBlockM * CTAS, BLOCK_N) : umma_idesc(kBlockM * CTAS, BLOCK_N, kFmt, kFmt);
      // Hands a barrier (same offset in every CTA of the pair) the completion of the UMMAs so far.
      auto commit_to = [&](uint64_t *bar) {
        if (!issuer) return;
        if constexpr (CTAS == 2) {
          umma_commit_pair_both(bar);
        } else {
          umma_commit(bar);
        }
      };
      // This loop is one thread feeding the tensor pipe, so its own instruction count is on the
      // critical path: every descriptor is the stage-0 descriptor plus a per-stage step (only the
      // 14-bit address field changes, and shared memory is below 2^18 bytes so it cannot carry).
      const uint64_t adesc0 = umma_desc_sw128(smem_u32(stage_a(0)));
      const uint64_t bdesc0 = umma_desc_sw128(smem_u32(stage_b(0)));
      const uint64_t sfa_desc0 = NVF4 ? umma_desc_sf(smem_u32(stage_sfa(0))) : 0;
      const uint64_t sfb_desc0 = NVF4 ? umma_desc_sf(smem_u32(stage_sfb(0))) : 0;
      constexpr uint64_t kStageStep = Cfg::kStageBytes >> 4;
      constexpr uint64_t kMmaStep = kMmaKBytes >> 4;
      constexpr uint64_t kSfTileStep = kSfTileBytes >> 4;
      (void)sfa_desc0;
      (void)sfb_desc0;
      (void)kSfTileStep;
      uint32_t sf_it = 0;  // NVFP4: K stages so far, over all tiles: picks the scale-factor set and its phase
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      WorkWalk walk(p, unit, num_units);
      WorkItem item;
      for (; ok && walk.next(&item); ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        // A tile that starts 64 rows into a 128-row scale group reads its B scale factors two
        // tensor-memory columns further on (32 rows per column).
        uint32_t sfb_skip = 0;
        if constexpr (NVF4) {
          int tm, tn;
          tile_coords(item.tile, p.tiles_m, p.tiles_n, &tm, &tn);
          sfb_skip = ((tn * BLOCK_N) % 128) / 32;
        }
        if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        const int kb_first = item.kb0;  // the item's first UMMA overwrites the accumulator
        for (int kb = item.kb0; kb < item.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, &abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t adesc = adesc0 + stage * kStageStep;
          const uint64_t bdesc = bdesc0 + stage * kStageStep;
          if constexpr (NVF4) {
            const uint32_t sf_set = sf_it & 1;
            const uint32_t sfa_tmem = tmem_base + Cfg::kAccCols + sf_set * Cfg::kSfSetCols;
            const uint32_t sfb_tmem = sfa_tmem + Cfg::kSfaCols;
            if (!mbar_wait(&sf_full_bar[sf_set], (sf_it >> 1) & 1, &abort_flag)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int j = 0; j < kMmasPerStage; ++j) {
              if constexpr (CTAS == 2) {
                if (issuer) umma_nvf4_ss_pair(d_tmem, adesc + j * kMmaStep, bdesc + j * kMmaStep, idesc, ((kb - kb_first) | j) != 0 ? 1u : 0u,
                                  sfa_tmem + j * 4, sfb_tmem + j * Cfg::kSfbColsPerMma + sfb_skip);
              } else {
                if (issuer) umma_nvf4_ss(d_tmem, adesc + j * kMmaStep, bdesc + j * kMmaStep, idesc, ((kb - kb_first) | j) != 0 ? 1u : 0u,
                             sfa_tmem + j * 4, sfb_tmem + j * Cfg::kSfbColsPerMma + sfb_skip);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < kMmasPerStage; ++j) {
              if constexpr (CTAS == 2) {
                if (issuer) umma_ss_pair<KIND>(d_tmem, adesc + j * kMmaStep, bdesc + j * kMmaStep, idesc, ((kb - kb_first) | j) != 0 ? 1u : 0u);
              } else {
                if (issuer) umma_ss<KIND>(d_tmem, adesc + j * kMmaStep, bdesc + j * kMmaStep, idesc, ((kb - kb_first) | j) != 0 ? 1u : 0u);
              }
            }
          }
          commit_to(&empty_bar[stage]);
          if constexpr (NVF4) {
            commit_to(&sf_empty_bar[sf_it & 1]);
            ++sf_it;
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        commit_to(&acc_full_bar[acc]);
      }
      if (!ok && issuer) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusMmaTimeout));
      }
    }
  } else if (NVF4 && warp == kPusherWarp0) {
    // ------------------------------------------------------------------ scale-factor copier (NVFP4)
    // One thread of the leader moves every stage's scale factors shared -> tensor memory, into
    // the set the MMAs are not reading, and hands the set over with a commit.
    if (lane == 0 && leader) {
      constexpr uint64_t kStageStep = Cfg::kStageBytes >> 4;
      constexpr uint64_t kSfTileStep = kSfTileBytes >> 4;
      const uint64_t sfa_desc0 = umma_desc_sf(smem_u32(stage_sfa(0)));
      const uint64_t sfb_desc0 = umma_desc_sf(smem_u32(stage_sfb(0)));
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;
      bool ok = true;
      WorkWalk walk(p, unit, num_units);
      WorkItem item;
      while (ok && walk.next(&item)) {
        for (int kb = item.kb0; kb < item.kb1; ++kb, ++it) {
          const uint32_t set = it & 1;
          if (!mbar_wait(&full_bar[stage], phase, &abort_flag) ||
              !mbar_wait(&sf_empty_bar[set], ((it >> 1) & 1) ^ 1, &abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t sfa_desc = sfa_desc0 + stage * kStageStep;
          const uint64_t sfb_desc = sfb_desc0 + stage * kStageStep;
          const uint32_t sfa_tmem = tmem_base + Cfg::kAccCols + set * Cfg::kSfSetCols;
          const uint32_t sfb_tmem = sfa_tmem + Cfg::kSfaCols;
#pragma unroll
          for (int j = 0; j < kMmasPerStage; ++j) {
            if constexpr (CTAS == 2) {
              tmem_cp_sf_pair(sfa_tmem + j * 4, sfa_desc + j * kSfTileStep);
            } else {
              tmem_cp_sf(sfa_tmem + j * 4, sfa_desc + j * kSfTileStep);
            }
#pragma unroll
            for (int g = 0; g < Cfg::kSfbGroups; ++g) {
              const uint64_t d = sfb_desc + (g * kMmasPerStage + j) * kSfTileStep;
              if constexpr (CTAS == 2) {
                tmem_cp_sf_pair(sfb_tmem + j * Cfg::kSfbColsPerMma + g * 4, d);
              } else {
                tmem_cp_sf(sfb_tmem + j * Cfg::kSfbColsPerMma + g * 4, d);
              }
            }
          }
          if constexpr (CTAS == 2) {
            umma_commit_pair_both(&sf_full_bar[set]);
          } else {
            umma_commit(&sf_full_bar[set]);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusMmaTimeout));
      }
    }
  } else if (B8 && warp >= kPusherWarp0) {
    // ------------------------------------------------------------------ converters (mixed form)
    // 16 e4m3 bytes of a row -> 16 halves = two 16-byte pieces of the row's 128 bytes in the
    // 128-byte swizzle (piece index xor row % 8). A warp's 32 lanes take 8 rows x 4 pieces: the
    // reads are 512 contiguous bytes, the writes touch every bank four times, which is the least
    // 512 bytes can.
    const int cw = static_cast<int>(warp) - kPusherWarp0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    WorkWalk walk(p, unit, num_units);
    WorkItem item;
    while (ok && walk.next(&item)) {
      for (int kb = item.kb0; kb < item.kb1; ++kb) {
        if (!mbar_wait(&raw_full_bar[stage], phase, &abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t *raw = stage_raw(stage);
        uint8_t *b16 = stage_b(stage);
#pragma unroll 4
        for (int piece = cw * 32 + static_cast<int>(lane); piece < Cfg::kBRows * 4; piece += kConverterWarps * 32) {
          const uint32_t r = static_cast<uint32_t>(piece) >> 2, q = static_cast<uint32_t>(piece) & 3;
          const uint4 v = *reinterpret_cast<const uint4 *>(raw + piece * 16);
          uint4 lo, hi;
          e4m3x4_to_f16x4(v.x, &lo.x, &lo.y);
          e4m3x4_to_f16x4(v.y, &lo.z, &lo.w);
          e4m3x4_to_f16x4(v.z, &hi.x, &hi.y);
          e4m3x4_to_f16x4(v.w, &hi.z, &hi.w);
          uint8_t *row_base = b16 + r * kRowBytes;
          *reinterpret_cast<uint4 *>(row_base + (((2 * q) ^ (r & 7)) << 4)) = lo;
          *reinterpret_cast<uint4 *>(row_base + (((2 * q + 1) ^ (r & 7)) << 4)) = hi;
        }
        fence_proxy_async_smem();  // the UMMA reads these bytes through the async proxy
        __syncwarp();
        if (lane == 0) {
          if (leader) {
            mbar_arrive(&full_bar[stage]);
          } else {
            mbar_arrive_remote(map_to_cta(smem_u32(&full_bar[stage]), 0));
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusProducerTimeout));
    }
  } else if (!B8 && warp >= kPusherWarp0) {
    // ------------------------------------------------------------------ pushers (scatter form)
    if (scatter && p.out_vector) {
      bool ok = true;
      int local = 0;
      const int pw = static_cast<int>(warp) - kPusherWarp0;
      const int col = static_cast<int>(lane) * 8;  // 8 elements = 16 bytes per lane, 512 bytes per row per warp
      WorkWalk walk(p, unit, num_units);
      WorkItem item;
      for (; ok && walk.next(&item); ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        int tm, tn;
        tile_coords(item.tile, p.tiles_m, p.tiles_n, &tm, &tn);
        const int m0 = tm * (kBlockM * CTAS) + static_cast<int>(cta_rank) * kBlockM;
        const int n0 = tn * BLOCK_N;
        if (!mbar_wait(&tile_done_bar[acc], acc_phase, &abort_flag)) {
          ok = false;
          break;
        }
        const bool col_ok = col < BLOCK_N && n0 + col < p.n;
        constexpr int kRowsInFlight = 8;
#pragma unroll 1
        for (int r0 = pw * kRowsInFlight; r0 < kBlockM; r0 += kPusherWarps * kRowsInFlight) {
          uint4 q[kRowsInFlight];
          bool live[kRowsInFlight];
#pragma unroll
          for (int i = 0; i < kRowsInFlight; ++i) {
            const int row = m0 + r0 + i;
            live[i] = col_ok && row < p.m;
            if (live[i]) {
              const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.out[0]) +
                                                                 static_cast<long long>(row) * p.out_ld + p.out_col0 + n0 + col);
              q[i] = __ldcg(src);  // from L2, where the epilogue's stores are
            }
          }
#pragma unroll
          for (int i = 0; i < kRowsInFlight; ++i) {
            if (live[i]) {
              const long long off = static_cast<long long>(m0 + r0 + i) * p.out_ld + p.out_col0 + n0 + col;
              for (int d = 1; d < p.num_out; ++d) {
                *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(p.out[d]) + off) = q[i];
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 2) {
            mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
          } else {
            mbar_arrive(&acc_empty_bar[acc]);
          }
        }
      }
      if (!ok && lane == 0) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusEpilogueTimeout));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    constexpr int HALF_N = Cfg::kHalfN;
    constexpr int HALF_CHUNKS = HALF_N / 32;
    const uint32_t quarter = warp & 3;  // which 32 lanes of tensor memory, i.e. which 32 rows of the tile
    const uint32_t half = warp >> 2;    // which share of the tile's columns (two halves; one whole in the mixed form)
    bool ok = true;
    int local = 0;
    const int is_bf16 = p.out_bf16;
    const bool has_cs_vec = p.col_scale != nullptr && !p.col_scale_scalar;
    const bool has_bias = p.bias != nullptr;
    const bool has_res = p.residual != nullptr;
    const bool has_gs = p.global_scale != nullptr;
    const float gscale = has_gs ? __ldg(p.global_scale) : 1.0f;
    const float cs_scalar = (p.col_scale && p.col_scale_scalar) ? __ldg(p.col_scale) : 1.0f;
    const bool out_vector = p.out_vector != 0;
    const bool res_vec_ok = has_res && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0 && (p.residual_ld % 8) == 0;
    float *cs_t = reinterpret_cast<float *>(smem + Cfg::kColParamOffset) + warp * 2 * HALF_N;
    float *bias_t = cs_t + HALF_N;
    const bool staged = p.out_staged != 0;
    uint8_t *obuf = smem + Cfg::kOutStageOffset + warp * Cfg::kOutStageBytesPerWarp;
    // Where this lane's row keeps its four 16-byte pieces in the warp's buffer (64-byte swizzle:
    // piece index xor bits 7-8 of the address), and where the pieces this lane fetches of other
    // lanes' rows go: piece (lane & 3) of rows (lane >> 2) + 8 i.
    const uint32_t own_row_off = lane * 64;
    const uint32_t own_swz = (lane >> 1) & 3;
    const uint32_t fetch_piece = lane & 3;
    const uint32_t fetch_row = lane >> 2;

    WorkWalk walk(p, unit, num_units);
    WorkItem item;
    for (; ok && walk.next(&item); ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      int tm, tn;
      tile_coords(item.tile, p.tiles_m, p.tiles_n, &tm, &tn);
      const int row = tm * (kBlockM * CTAS) + static_cast<int>(cta_rank) * kBlockM + quarter * 32 + lane;
      const int n0 = tn * BLOCK_N + half * HALF_N;  // first column this warp owns

      // This warp's per-column scale and bias, widened to fp32 once, in its own slice of shared
      // memory.
      if (has_cs_vec || has_bias) {
        __syncwarp();  // the previous tile's reads are done
        // (with row groups, the tile's group picks the row of the (groups, n) scales and bias)
        const long long goff = p.rows_per_group > 0 ? static_cast<long long>((tm * (kBlockM * CTAS)) / p.rows_per_group) * p.n : 0;
        for (int i = lane; i < HALF_N; i += 32) {
          const int n = n0 + i;
          cs_t[i] = (has_cs_vec && n < p.n) ? __ldg(p.col_scale + goff + n) : 1.0f;
          bias_t[i] = (has_bias && n < p.n) ? load16(p.bias, goff + n, is_bf16) : 0.0f;
        }
        __syncwarp();
      }

      if (!mbar_wait(&acc_full_bar[acc], acc_phase, &abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const bool row_ok = row < p.m;
      const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
      const float rs_cs = rs * cs_scalar;
      const long long res_row =
          (has_res && row_ok) ? static_cast<long long>(row % p.residual_rows) * p.residual_ld : 0;
      const long long out_off = static_cast<long long>(row) * p.out_ld + p.out_col0;
      int chunks = (p.n - n0 + 31) / 32;  // chunks of this warp's half that hold a valid column
      chunks = chunks < 0 ? 0 : (chunks > HALF_CHUNKS ? HALF_CHUNKS : chunks);
      const uint32_t tacc = tmem_base + ((quarter * 32) << 16) + acc * BLOCK_N + half * HALF_N;

      // The largest magnitude among a chunk's 32 rounded results of this lane's row, merged into the
      // row's maximum in global memory. Magnitudes of one 16-bit format order like their bit
      // patterns, and non-negative floats like theirs, so both maxima are integer ones.
      auto note_row_amax = [&](const uint32_t (&packed)[16], int nc) {
        uint32_t top = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (nc + 2 * j < p.n) top = max(top, max(packed[j] & 0x7fffu, (packed[j] >> 16) & 0x7fffu));
        }
        const float as_float = is_bf16 ? __uint_as_float(top << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(top)));
        atomicMax(reinterpret_cast<unsigned int *>(p.row_amax) + row, __float_as_uint(as_float));
      };
      // One 32-column chunk: scale, bias, activation, residual in fp32; one rounding; store.
      auto finish_chunk = [&](int c, uint32_t (&v)[32]) {
        const int nc = n0 + c * 32;
        float x[32];
        // Staged form: once the store of the chunk before has read the warp's buffer, the
        // residual's 32 rows x 64 bytes are fetched into it with four coalesced 16-byte copies per
        // lane (8 rows x 64 bytes per instruction) that bypass the registers; the arithmetic below
        // runs while they are on their way.
        if (staged) {
          if (lane == 0) bulk_wait_group_read0();
          __syncwarp();
          if (has_res) {
            const int col = nc + static_cast<int>(fetch_piece) * 8;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t r = i * 8 + fetch_row;
              const int grow = row - static_cast<int>(lane) + static_cast<int>(r);
              const bool live = grow < p.m && col < p.n;
              const uint16_t *src = reinterpret_cast<const uint16_t *>(p.residual) +
                                    (live ? static_cast<long long>(grow) * p.residual_ld + col : 0);
              cp_async_16(obuf + r * 64 + ((fetch_piece ^ ((r >> 1) & 3)) << 4), src, live ? 16u : 0u);
            }
          }
        }
        if (has_cs_vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 s4 = *reinterpret_cast<const float4 *>(cs_t + c * 32 + j);
            x[j] = __uint_as_float(v[j]) * (rs * s4.x);
            x[j + 1] = __uint_as_float(v[j + 1]) * (rs * s4.y);
            x[j + 2] = __uint_as_float(v[j + 2]) * (rs * s4.z);
            x[j + 3] = __uint_as_float(v[j + 3]) * (rs * s4.w);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]) * rs_cs;
        }
        if (has_gs) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] *= gscale;
        }
        if (has_bias) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 b4 = *reinterpret_cast<const float4 *>(bias_t + c * 32 + j);
            x[j] += b4.x;
            x[j + 1] += b4.y;
            x[j + 2] += b4.z;
            x[j + 3] += b4.w;
          }
        }
        if (p.act == kActGeluTanh) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = gelu_tanh(x[j]);
        }
        if (staged) {
          if (has_res) {
            cp_async_wait_all();
            __syncwarp();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint4 q = *reinterpret_cast<const uint4 *>(obuf + own_row_off + ((g ^ own_swz) << 4));
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                if (is_bf16) {
                  x[g * 8 + 2 * h] += __uint_as_float(w[h] << 16);
                  x[g * 8 + 2 * h + 1] += __uint_as_float(w[h] & 0xffff0000u);
                } else {
                  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[h]));
                  x[g * 8 + 2 * h] += f.x;
                  x[g * 8 + 2 * h + 1] += f.y;
                }
              }
            }
            // (a lane's row is read by that lane only, so it may be overwritten without another barrier)
          }
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) packed[j] = pack16(x[2 * j], x[2 * j + 1], is_bf16);
          if (p.row_amax != nullptr && row_ok) note_row_amax(packed, nc);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            *reinterpret_cast<uint4 *>(obuf + own_row_off + ((g ^ own_swz) << 4)) =
                make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          // Rows past m and columns past n are not written: the tensor map ends there.
          if (lane == 0) {
            for (int d = 0; d < p.num_out; ++d) tma_store_2d(&tmaps_out.at[d], obuf, nc, row - static_cast<int>(lane));
            bulk_commit_group();
          }
          return;
        }
        if (has_res && row_ok) {
          if (res_vec_ok) {
            const uint4 *rp = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.residual) + res_row + nc);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (nc + g * 8 < p.n) {  // n is a multiple of 8: a group of 8 is whole or absent
                const uint4 q = rp[g];
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  if (is_bf16) {
                    x[g * 8 + 2 * h] += __uint_as_float(w[h] << 16);
                    x[g * 8 + 2 * h + 1] += __uint_as_float(w[h] & 0xffff0000u);
                  } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[h]));
                    x[g * 8 + 2 * h] += f.x;
                    x[g * 8 + 2 * h + 1] += f.y;
                  }
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (nc + j < p.n) x[j] += load16(p.residual, res_row + nc + j, is_bf16);
            }
          }
        }
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) packed[j] = pack16(x[2 * j], x[2 * j + 1], is_bf16);
        if (!row_ok) return;
        if (p.row_amax != nullptr) note_row_amax(packed, nc);
        // (In the scatter form the peers' copies are made by the pusher warps from this one.)
        {
          uint16_t *out_row = reinterpret_cast<uint16_t *>(p.out[0]) + out_off;
          if (out_vector) {
            // 64 contiguous bytes of this thread's row, as four 16-byte stores.
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (nc + g * 8 < p.n) {  // n is a multiple of 8: a group of 8 is whole or absent
                *reinterpret_cast<uint4 *>(out_row + nc + g * 8) =
                    make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (nc + j < p.n) {
                out_row[nc + j] = static_cast<uint16_t>((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffff));
              }
            }
          }
        }
      };

      uint32_t va[32], vb[32];
      if (item.partial) {
        // Part of a tile's K range (the stream-K rounds): this warp's 32 rows x HALF_N columns of
        // the accumulator go to the workspace as they are, the accumulator is handed back, and
        // the warp counts itself in. The tile has exactly two parts; whichever warp comes second
        // adds them, head first, and finishes the sum like any other accumulator. A partial lies
        // chunk by chunk, four columns of 32 rows to a 512-byte line, so every store and load of
        // a warp is one contiguous line.
        constexpr int kWarpFloats = HALF_N * 32;
        constexpr int kSlotFloats = CTAS * kEpilogueWarps * kWarpFloats;  // one unit's part of one tile
        const int within = (static_cast<int>(cta_rank) * kEpilogueWarps + static_cast<int>(warp)) * kWarpFloats;
        float *mine = p.sk_partials + (static_cast<long long>(unit) * 2 + (item.head ? 1 : 0)) * kSlotFloats + within;
        // The other part: the tile's head belongs to the unit before the one that holds its tail
        // (slot 1 of that unit), the tail to the unit after (its slot 0).
        const float *other = p.sk_partials +
                             (static_cast<long long>(item.head ? unit + 1 : unit - 1) * 2 + (item.head ? 0 : 1)) * kSlotFloats + within;
        uint32_t *counter = p.sk_counters + (item.sk_tile * CTAS + static_cast<int>(cta_rank)) * kEpilogueWarps + warp;
        // Has the other holder counted itself in already? (It has when this is a tail, a unit's
        // last item: the tile's head was the first thing its holder did in this part of the
        // schedule.) Then this warp's part never goes to memory: the other part is added to the
        // accumulator as it comes out of tensor memory.
        uint32_t there = 0;
        if (lane == 0) there = *reinterpret_cast<volatile uint32_t *>(counter);
        there = __shfl_sync(0xffffffffu, there, 0);
        if (there != 0) {
          __threadfence();  // the other part's stores are ordered before its count, which was just read
          float4 pre[8];
          const float4 *op = reinterpret_cast<const float4 *>(other) + lane;
          if (chunks > 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) pre[j] = __ldcg(op + j * 32);
          }
#pragma unroll 1
          for (int c = 0; c < chunks; ++c) {
            tmem_ld_32x32(tacc + c * 32, va);
            tmem_ld_wait(va);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              // head + tail in that order, whichever of the two this warp holds (the sum is the same
              // either way round, bit for bit)
              va[4 * j] = __float_as_uint(__fadd_rn(__uint_as_float(va[4 * j]), pre[j].x));
              va[4 * j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(va[4 * j + 1]), pre[j].y));
              va[4 * j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(va[4 * j + 2]), pre[j].z));
              va[4 * j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(va[4 * j + 3]), pre[j].w));
            }
            if (c + 1 < chunks) {
#pragma unroll
              for (int j = 0; j < 8; ++j) pre[j] = __ldcg(op + (c + 1) * 256 + j * 32);
            }
            finish_chunk(c, va);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2) {
              mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
            } else {
              mbar_arrive(&acc_empty_bar[acc]);
            }
            *counter = 0;  // ready for the next launch
          }
          continue;
        }
        tmem_ld_32x32(tacc, va);
#pragma unroll 1
        for (int c = 0; c < HALF_CHUNKS; ++c) {
          tmem_ld_wait(va);
          float4 *dst = reinterpret_cast<float4 *>(mine + c * 1024) + lane;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dst[j * 32] = make_float4(__uint_as_float(va[4 * j]), __uint_as_float(va[4 * j + 1]), __uint_as_float(va[4 * j + 2]),
                                      __uint_as_float(va[4 * j + 3]));
          }
          if (c + 1 < HALF_CHUNKS) tmem_ld_32x32(tacc + (c + 1) * 32, va);
        }
        tc_fence_before_sync();
        __threadfence();  // this lane's part of the partial is visible before the count below says so
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) {
          if constexpr (CTAS == 2) {
            mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
          } else {
            mbar_arrive(&acc_empty_bar[acc]);
          }
          arrived = atomicAdd(counter, 1u);
        }
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == 0) continue;  // the other holder of this tile will finish it
        __threadfence();
        const float *head_part = item.head ? mine : other;
        const float *tail_part = item.head ? other : mine;
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          const float4 *hp = reinterpret_cast<const float4 *>(head_part + c * 1024) + lane;
          const float4 *tp = reinterpret_cast<const float4 *>(tail_part + c * 1024) + lane;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 h4 = __ldcg(hp + j * 32);
            const float4 t4 = __ldcg(tp + j * 32);
            va[4 * j] = __float_as_uint(__fadd_rn(h4.x, t4.x));
            va[4 * j + 1] = __float_as_uint(__fadd_rn(h4.y, t4.y));
            va[4 * j + 2] = __float_as_uint(__fadd_rn(h4.z, t4.z));
            va[4 * j + 3] = __float_as_uint(__fadd_rn(h4.w, t4.w));
          }
          finish_chunk(c, va);
        }
        __syncwarp();
        if (lane == 0) *counter = 0;  // ready for the next launch
        continue;
      }

      // Tensor-memory loads run one chunk ahead of the arithmetic.
      const int chunks_run = chunks;
      if (chunks_run > 0) tmem_ld_32x32(tacc, va);
#pragma unroll 1
      for (int c = 0; c < chunks_run; c += 2) {
        tmem_ld_wait(va);
        if (c + 1 < chunks_run) tmem_ld_32x32(tacc + (c + 1) * 32, vb);
        finish_chunk(c, va);
        if (c + 1 < chunks_run) {
          tmem_ld_wait(vb);
          if (c + 2 < chunks_run) tmem_ld_32x32(tacc + (c + 2) * 32, va);
          finish_chunk(c + 1, vb);
        }
      }
      tc_fence_before_sync();
      if (scatter) __threadfence();  // the tile's stores are visible before the pushers are told
      __syncwarp();
      if (lane == 0) {
        if (scatter) mbar_arrive(&tile_done_bar[acc]);
        if constexpr (CTAS == 2) {
          mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
        } else {
          mbar_arrive(&acc_empty_bar[acc]);
        }
      }
    }
    if (staged && lane == 0) bulk_wait_group0();  // this warp's stores have left its buffer and landed
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusEpilogueTimeout));
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag != 0) {
    // A wait gave up. Give loads that may still be in flight time to land before the shared
    // memory and tensor memory they target are released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  // In a pair the leader's UMMAs read the other CTA's shared memory and both CTAs signal each
  // other's barriers, so neither may leave or free tensor memory before both are done.
  if constexpr (CTAS == 2) cluster_sync_all();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc<CTAS>(tmem_base, Cfg::kTmemCols);
  }
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// A (rows, row_bytes) byte matrix cut into boxes of (box_rows, 128 bytes) in the 128-byte swizzle.
bool make_tmap(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// An e4m3 (rows, k) weight read in boxes of (box_rows, 64 bytes), as it lies (no swizzle): the
// converter warps of the mixed form re-lay it.
bool make_tmap_raw(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The scale-factor tiles of one operand as a (tiles, 512 byte) matrix of 32-bit words, read in
// boxes of kMmasPerStage tiles (the factors of one K stage of one 128-row group), unswizzled.
bool make_tmap_sf(CUtensorMap *map, const void *base, uint64_t tiles) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {kSfTileBytes / 4, tiles};
  cuuint64_t strides[1] = {kSfTileBytes};
  cuuint32_t box[2] = {kSfTileBytes / 4, static_cast<cuuint32_t>(kMmasPerStage)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The (m, n) matrix of 16-bit results with `ld` elements between rows, written in boxes of 32 rows
// x 32 columns (64 bytes) from shared memory in the 64-byte swizzle.
bool make_tmap_out(CUtensorMap *map, void *base, uint64_t m, uint64_t n, uint64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {n, m};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int KIND, int BLOCK_N, int CTAS, bool B8 = false>
cudaError_t launch_one(const GemmArgs &a, KernelParams kp, uint64_t row_bytes, const char **why) {
  using Cfg = Config<BLOCK_N, KIND == kKindNvf4, CTAS, B8>;
  kp.tiles_m = (a.m + kBlockM * CTAS - 1) / (kBlockM * CTAS);
  kp.tiles_n = (a.n + BLOCK_N - 1) / BLOCK_N;
  CUtensorMap ta, tb;
  const bool b_ok = B8 ? make_tmap_raw(&tb, a.b, a.n, row_bytes / 2, Cfg::kBRows) : make_tmap(&tb, a.b, a.n, row_bytes, Cfg::kBRows);
  if (!make_tmap(&ta, a.a, a.m, row_bytes, kBlockM) || !b_ok) {
    *why = "cuTensorMapEncodeTiled refused the operand";
    return cudaErrorInvalidValue;
  }
  CUtensorMap tsfa = ta, tsfb = tb;  // only dereferenced by the block-scaled kind
  if constexpr (KIND == kKindNvf4) {
    const uint64_t k_tiles = static_cast<uint64_t>(a.sf_k_tiles);
    if (!make_tmap_sf(&tsfa, a.sfa, static_cast<uint64_t>((a.m + 127) / 128) * k_tiles) ||
        !make_tmap_sf(&tsfb, a.sfb, static_cast<uint64_t>((a.n + 127) / 128 + 1) * k_tiles)) {
      *why = "cuTensorMapEncodeTiled refused the scale factors";
      return cudaErrorInvalidValue;
    }
  }
  // Results leave through per-warp shared-memory buffers and TMA stores when the destination can
  // be described by a tensor map (one 16-byte aligned matrix, pitch a multiple of 8 elements) and
  // the residual, if any, is a plain 16-byte aligned matrix of out's rows; otherwise every lane
  // stores (and loads the residual of) its own row.
  OutMaps tout;
  for (int d = 0; d < kMaxGemmOutputs; ++d) tout.at[d] = ta;
  kp.out_staged = 0;
  if (kp.out_vector && !a.no_staged_out && (!kp.residual || (kp.residual_rows == a.m && (reinterpret_cast<uintptr_t>(kp.residual) & 15) == 0 &&
                                         kp.residual_ld % 8 == 0))) {
    kp.out_staged = 1;
    for (int d = 0; d < kp.num_out && kp.out_staged; ++d) {
      void *base = reinterpret_cast<uint16_t *>(kp.out[d]) + kp.out_col0;
      if (!make_tmap_out(&tout.at[d], base, a.m, a.n, kp.out_ld)) kp.out_staged = 0;
    }
  }
  auto kernel = gemm_tn_kernel<KIND, BLOCK_N, CTAS, B8>;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      *why = "cudaFuncSetAttribute(max dynamic shared memory) failed";
      return e;
    }
    attr_set = true;
  }
  const int tiles = kp.tiles_m * kp.tiles_n;
  const size_t part_floats_per_unit = static_cast<size_t>(2) * CTAS * kBlockM * BLOCK_N;
  const bool may_stream_k = a.sk_partials && a.sk_counters && !a.no_stream_k && (kp.num_out == 1 || kp.out_staged) &&
                            part_floats_per_unit * (sm_count() / CTAS) <= a.sk_partial_floats &&
                            static_cast<size_t>(2) * sm_count() * kMaxEpilogueWarps <= a.sk_counter_words;
  const GemmSchedule sch = gemm_schedule(tiles, sm_count() / CTAS, kp.num_kb, may_stream_k);
  const int units = sch.units;
  kp.dp_rounds = sch.dp_rounds;
  kp.sk_tiles = sch.sk_tiles;
  kp.sk_first_tile = sch.sk_first_tile;
  kp.sk_partials = sch.sk_tiles ? a.sk_partials : nullptr;
  kp.sk_counters = sch.sk_tiles ? a.sk_counters : nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(units * CTAS), 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Programmatic dependent launch: the prologue may run while the previous kernel drains.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tsfa, tsfb, tout, kp);
  if (e != cudaSuccess) *why = "kernel launch failed";
  return e;
}

}  // namespace

int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
      cached = n;
    } else {
      cached = 148;
    }
  }
  return cached;
}

// The schedule (see the head of this file). What the stream-K part can save is the idle share of
// the last round, (units - remainder) / units of a tile's main loop; what it costs, measured, is
// about ten microseconds of a launch (two more epilogue-side passes per unit, the second of them
// exposed at the end), that is some thirty K stages. It is used where the saving is forty stages
// or more: long-K products whose last round is poorly filled (8704 x 3072 x 12288: 408 tiles on 74
// pairs, 248 -> 232 us); with 3072-deep tiles it never is. A product with fewer tiles than half
// the units and a long K has every tile cut into two halves on twice as many units (the same two
// holders per tile, the same workspace slots and counters).
GemmSchedule gemm_schedule(int tiles, int max_units, int num_kb, bool allow_stream_k) {
  GemmSchedule s = {};
  s.units = tiles < max_units ? tiles : max_units;
  if (s.units < 1) s.units = 1;
  const int full_rounds = tiles / s.units;
  const int remainder = tiles % s.units;
  const long long saved_stages = static_cast<long long>(s.units - remainder) * num_kb / s.units;
  if (allow_stream_k && 2 * tiles <= max_units && num_kb / 2 >= kStreamKMinSavedStages) {
    // Fewer tiles than half the units and a long K: every tile is cut in two halves of its K
    // stages, held by two neighbouring units (4352 x 384 x 12288: 34 tiles on 68 of 74 pairs).
    s.units = 2 * tiles;
    s.dp_rounds = 0;
    s.sk_tiles = tiles;
    s.sk_first_tile = 0;
  } else if (allow_stream_k && full_rounds >= 1 && remainder > 0 && saved_stages >= kStreamKMinSavedStages) {
    s.dp_rounds = full_rounds - 1;
    s.sk_tiles = remainder + s.units;
    s.sk_first_tile = s.dp_rounds * s.units;
  } else {
    s.dp_rounds = (tiles + s.units - 1) / s.units;
  }
  return s;
}

// Which kernel a product runs on, and its schedule; host arithmetic only.
void gemm_plan(GemmKind kind, int m, int n, int k, int sms, int allow_stream_k, int *plan) {
  const int row_bytes = kind == kGemmE4M3 ? k : kind == kGemmNvf4 ? k / 2 : k * 2;
  const int num_kb = (row_bytes + kRowBytes - 1) / kRowBytes;
  const bool pair = m > kBlockM && n > 128;
  const bool skinny = m <= kBlockM && (n + 255) / 256 < sms;
  const int ctas = pair ? 2 : 1;
  const int block_n = kind == kGemmNvf4 ? 192 : (pair ? 256 : ((n <= 128 || skinny) ? 128 : 256));
  const int tiles = ((m + kBlockM * ctas - 1) / (kBlockM * ctas)) * ((n + block_n - 1) / block_n);
  const GemmSchedule s = gemm_schedule(tiles, sms / ctas, num_kb, allow_stream_k != 0);
  plan[0] = ctas, plan[1] = block_n, plan[2] = tiles, plan[3] = num_kb;
  plan[4] = s.units, plan[5] = s.dp_rounds, plan[6] = s.sk_tiles, plan[7] = s.sk_first_tile;
}

// Two parts per SM of 128 rows x 256 columns at most; a counter per epilogue warp of every tile of
// the stream-K part, which has fewer than two rounds of tiles.
size_t gemm_stream_k_partial_floats() { return static_cast<size_t>(sm_count()) * 2 * kBlockM * 256; }
size_t gemm_stream_k_counter_words() { return static_cast<size_t>(sm_count()) * 2 * kMaxEpilogueWarps; }

cudaError_t launch_gemm(const GemmArgs &a, const char **why) {
  *why = "";
  uint64_t row_bytes;
  switch (a.kind) {
    case kGemmF16:
    case kGemmBF16: row_bytes = static_cast<uint64_t>(a.k) * 2; break;
    case kGemmE4M3: row_bytes = static_cast<uint64_t>(a.k); break;
    default: row_bytes = static_cast<uint64_t>(a.k) / 2; break;
  }
  if (a.m <= 0 || a.n <= 0 || a.k <= 0 || row_bytes % 16 != 0 || a.n % 8 != 0) {
    *why = "shape the kernels cannot read (rows of 16 bytes, n a multiple of 8)";
    return cudaErrorInvalidValue;
  }
  if ((reinterpret_cast<uintptr_t>(a.a) & 15) || (reinterpret_cast<uintptr_t>(a.b) & 15)) {
    *why = "operand base is not 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  if (a.rows_per_group != 0 && (a.rows_per_group < 0 || a.rows_per_group % 256 != 0 || a.col_scale_scalar)) {
    *why = "row groups are multiples of 256 rows with one scale per channel";
    return cudaErrorInvalidValue;
  }
  KernelParams kp;
  kp.m = a.m;
  kp.n = a.n;
  kp.num_kb = static_cast<int>((row_bytes + kRowBytes - 1) / kRowBytes);
  kp.tiles_m = kp.tiles_n = 0;  // set per instantiation
  kp.sfa = a.sfa;
  kp.sfb = a.sfb;
  kp.sf_k_tiles = a.sf_k_tiles;
  kp.row_scale = a.row_scale;
  kp.col_scale = a.col_scale;
  kp.col_scale_scalar = a.col_scale_scalar;
  kp.global_scale = a.global_scale;
  kp.bias = a.bias;
  kp.residual = a.residual;
  kp.residual_rows = a.residual_rows > 0 ? a.residual_rows : a.m;
  kp.rows_per_group = a.rows_per_group;
  kp.residual_ld = a.residual_ld;
  kp.act = a.act;
  kp.row_amax = a.row_amax;
  kp.out_bf16 = a.out_bf16;
  kp.num_out = 0;
  kp.out[kp.num_out++] = a.out;
  for (int i = 0; i < a.num_extra_out && kp.num_out < kMaxGemmOutputs; ++i) {
    if (a.extra_out[i]) kp.out[kp.num_out++] = a.extra_out[i];
  }
  for (int i = kp.num_out; i < kMaxGemmOutputs; ++i) kp.out[i] = nullptr;
  kp.out_ld = a.out_ld > 0 ? a.out_ld : a.n;
  kp.out_col0 = a.out_ld > 0 ? a.out_col0 : 0;
  kp.out_vector = (kp.out_ld % 8 == 0 && kp.out_col0 % 8 == 0) ? 1 : 0;
  for (int i = 0; i < kp.num_out; ++i) {
    if (reinterpret_cast<uintptr_t>(kp.out[i]) & 15) kp.out_vector = 0;
  }
  if (kp.num_out > 1 && !kp.out_vector) {
    *why = "scatter destinations need 16-byte aligned bases and a pitch and column offset that are multiples of 8";
    return cudaErrorInvalidValue;
  }
  kp.status = a.status;
  if (a.b_is_e4m3 && (a.kind != kGemmF16 || kp.num_out > 1)) {
    *why = "an e4m3 right operand widened in the kernel goes with half operands and one destination";
    return cudaErrorInvalidValue;
  }

  // A pair of CTAs per 256-row tile halves the B bytes each SM pulls from L2; it needs two row
  // blocks to share the B tile between. Narrow outputs use the narrower single-CTA tile so that
  // fewer columns of the MMA are padding.
  const bool pair = a.m > kBlockM && a.n > 128 && !a.force_single_cta;
  // One row block (the skinny case: decode rows, adaLN modulation) is bound by streaming the
  // weight from HBM, so what matters is how many SMs pull on it: 128-wide tiles give twice as
  // many CTAs as 256-wide ones until the grid is full.
  const bool skinny = a.m <= kBlockM && (a.n + 255) / 256 < sm_count();
  if (a.kind == kGemmNvf4) {
    if ((reinterpret_cast<uintptr_t>(a.sfa) & 15) || (reinterpret_cast<uintptr_t>(a.sfb) & 15)) {
      *why = "scale-factor base is not 16-byte aligned";
      return cudaErrorInvalidValue;
    }
    return pair ? launch_one<kKindNvf4, 192, 2>(a, kp, row_bytes, why) : launch_one<kKindNvf4, 192, 1>(a, kp, row_bytes, why);
  }
  const bool narrow = a.n <= 128 || skinny;
  switch (a.kind) {
    case kGemmE4M3:
      if (pair) return launch_one<kKindF8, 256, 2>(a, kp, row_bytes, why);
      return narrow ? launch_one<kKindF8, 128, 1>(a, kp, row_bytes, why) : launch_one<kKindF8, 256, 1>(a, kp, row_bytes, why);
    case kGemmBF16:
      if (pair) return launch_one<kKindBF16, 256, 2>(a, kp, row_bytes, why);
      return narrow ? launch_one<kKindBF16, 128, 1>(a, kp, row_bytes, why) : launch_one<kKindBF16, 256, 1>(a, kp, row_bytes, why);
    default:
      if (a.b_is_e4m3) {
        if (pair) return launch_one<kKindF16, 256, 2, true>(a, kp, row_bytes, why);
        return narrow ? launch_one<kKindF16, 128, 1, true>(a, kp, row_bytes, why)
                      : launch_one<kKindF16, 256, 1, true>(a, kp, row_bytes, why);
      }
      if (pair) return launch_one<kKindF16, 256, 2>(a, kp, row_bytes, why);
      return narrow ? launch_one<kKindF16, 128, 1>(a, kp, row_bytes, why) : launch_one<kKindF16, 256, 1>(a, kp, row_bytes, why);
  }
}

}  // namespace flsm100
