// Frozen-base K-quant projection GEMMs on the sm_100a tensor cores.
//
//   forward   out[T, N]  = act[T, K] * W[N, K]^T (+ bias) (+ lora_act[T, r] * B[r, N])
//   backward  out[T, K] += act[T, N] * W[N, K]            (+ lora_act[T, r] * A[K, r]^T)
//
// Replaces the CUDA-core kernels gemm_q4_k_batch / gemm_q6_k_batch (Glacier.Inference fatbin, launched at
// src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:83-129) and gemm_q4_k_bwd / gemm_q6_k_bwd
// (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:193-332), and folds in the rank-r products that the reference runs
// on the host (src/Glacier.Tune/Kernels/LoraKernels.cs:57-86,296-339).
//
// One CTA owns 128 weight rows (forward) or 128 weight columns (backward) and ALL tokens of its token chunk
// (up to 512), so each weight is dequantized once per CTA and reused by every token:
//   D[128 x tokens] (TMEM, fp32)  +=  Wtile[128 x 64] (SMEM, dequantized 16-bit)  x  act[tokens x 64]^T (SMEM via TMA)
//
// Warp roles (640 threads):
//   warp 0        TMA producer of the packed half-super-blocks of W (raw bytes)
//   warp 19       TMA producer of the 16-bit activation tiles
//   warps 1, 18   tcgen05.mma issuers (one thread each, alternate stages, a turn token keeps the order fixed);
//                 warp 1 owns the TMEM allocation
//   warps 2-17    four groups of 4 warps that dequantize every fourth operand stage each (raw blocks -> 128-byte-
//                 swizzled tiles); afterwards all 16 run the epilogue (tcgen05.ld -> bias -> global store / atomic add)
//
// One launch serves up to three member projections (forward: they share the activation tiles, each tile index belongs
// to one member; backward: their contraction ranges are concatenated and all sum into one dX), each with its own
// rank-update stage when it has an adapter.  The dual forward (Params.dual) is the gate | up launch of a SwiGLU block:
// every tile holds 64 rows of both members, interleaved so that one warp reads gate and up of a feature from its own
// TMEM quadrant, and the epilogue writes SiLU(gate) * up as 16-bit values (gate and up themselves only where wanted).
//
// The dequantized tile image is the same for both directions: row = weight row n, 128 bytes = 64 consecutive
// k, chunks XOR-swizzled by (row & 7).  Forward reads it as a K-major A operand (M = n, K = k); backward
// reads it as an MN-major A operand (M = k, K = n) - no transposed copy of W is ever formed.
//
// Every mbarrier wait is bounded (wall-clock limit); on a timeout the CTA records a code in status[0], all
// roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "gt_internal.h"
#include "gt_ptx.cuh"
#include "gt_quant.cuh"

namespace gt {

namespace {

constexpr int kTileW = 128;        // weight rows (forward) / columns (backward) per CTA = UMMA M per CTA
constexpr int kChunk = 64;         // contraction elements per operand stage (one 128-byte row)
constexpr int kMaxTok = 512;       // tokens per CTA = TMEM columns
constexpr int kAStageBytes = kTileW * kChunk * 2;   // 16 KiB
constexpr int kNumA = 4;            // operand stages (dequantized weight tile + activation tile)
// Shared memory of a CTA: [activation stages | dequantized weight stages | ring of packed weight blocks | barriers].
// An activation stage holds XROWS token rows of 128 bytes (a kernel template parameter: 256 rows, or 128 in the
// few-token variant).  Raw (still packed) weight blocks come from HBM, whose latency under load is several operand-stage
// times (about 2.5 k clocks): the raw ring gets all the shared memory that is left, cut into as many stages as the
// format's stage size allows (up to kMaxRaw) - 32 KB beside 256-row activation stages, 96 KB beside 128-row ones,
// where nothing but the bytes in flight bounds the kernel.
constexpr int kOffX = 0;
constexpr int kOffBar = kNumA * 32768 + kNumA * kAStageBytes + 32768;
constexpr int kMaxRaw = 16;
constexpr int kBarBytes = 512;
constexpr int kDequantWarps = 16;   // four groups of 4
constexpr int kThreads = 32 * (4 + kDequantWarps);   // + weight producer (0), two MMA issuers (1, 18), activation producer (19)
constexpr int kIssuer2Warp = 18, kActProducerWarp = 19;
constexpr int kSmemBytes = kOffBar + kBarBytes + 1024;   // + slack for 1024-byte alignment

// barrier slots (8 bytes each) inside the kOffBar region
// (an operand stage = dequantized weight tile + activation tile; both share one slot index and one full/empty pair)
constexpr int kMaxRawBars = 24;     // (slot, class) barriers of the raw ring, see kCls in the kernel
constexpr int kBarRawFull = 0, kBarRawEmpty = kMaxRawBars, kBarFull = 2 * kMaxRawBars, kBarEmpty = kBarFull + kNumA,
              kBarAcc = kBarEmpty + kNumA, kBarTurn = kBarAcc + 1, kNumBars = kBarTurn + 2;
constexpr int kOffTmemSlot = kNumBars * 8;       // u32
constexpr int kOffAbort = kOffTmemSlot + 4;      // int
static_assert(kOffAbort + 4 <= kBarBytes, "barrier region too small");

// One launch serves up to kMaxMembers projections that share their input (forward: q,k,v or gate,up read the same X,
// each writes its own Y) or their output (backward: dX += sum over members of dY_m * W_m).
constexpr int kMaxMembers = 3;
struct Member {
    CUtensorMap tm_hdr, tm_q0, tm_q1;   // packed weight bytes of this member
    CUtensorMap tm_act;                 // backward: this member's 16-bit dY; forward: member 0 holds the shared X
    float *out;                         // forward: this member's Y; backward: the shared dX (member 0 is read)
    const float *bias;
    const float *lora_w;                // forward: B [R, N]; backward: A [K, R]
    const float *lora_act;              // fp32 [T, R]: X*A (forward) or dY*B^T (backward); scaled by lora_scale in the kernel
    const int *lora_flag;
    float lora_scale;
    int row_base;                       // first weight row of the window this launch works on (0: the whole tensor)
    int rank, N, ld_out;
    int first, count;                   // forward: first tile / tiles of this member; backward: first unit / units
};
struct Params {
    Member m[kMaxMembers];
    int n_members;
    int *status;
    long long *trace;   // optional timeline of CTA (0,0,0): [12 rows][128] SM clock values, or null
    int T, K;
    int t_box;       // token rows per activation TMA box
    int splits, units;
    int atomic_out;  // 1: red.add into out, 0: plain store (forward: + bias)
    int tmem_cols;
    int par_ok;      // 0: keep the two MMA issuers on the turn token at every token count (GT_MMA_PAR=0)
    // Dual forward (gate | up with the SwiGLU product in the epilogue; replaces gemm_q4_k_swiglu_batch,
    // src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:152-183): two members of the same shape, no split-K.  A CTA's tile
    // holds 64 rows of member 0 and the SAME 64 rows of member 1, laid out so that TMEM lanes 32 q + l and 32 q + 16 + l
    // (l < 16) are the two members' row 16 q + l: one warp shuffle brings gate and up of a feature together.
    int dual;
    void *h16;       // T16 [T, ld_h16]: SiLU(gate) * up, or null
    int ld_h16;
};
// dual forward: row r of the packed-weight stage (member r / 64, feature r % 64) -> row of the operand tile / TMEM lane
__host__ __device__ inline int dual_row(int r) { return ((r & 63) >> 4) * 32 + (r >> 6) * 16 + (r & 15); }

// status codes written on a bounded-wait timeout: 100*role + barrier kind
enum { kCodeProducer = 100, kCodeMma = 200, kCodeDequant = 300, kCodeEpilogue = 400 };

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int n) {
        if (++idx == n) {
            idx = 0;
            phase ^= 1u;
        }
    }
};

// PAIR = false: one CTA per tile, tcgen05 cta_group::1, M = 128.
// PAIR = true : a cluster of two CTAs (the two SMs of a TPC) works on two adjacent tiles with cta_group::2 MMAs of
//               M = 256.  Each CTA dequantizes its own 128 weight rows and loads only HALF of the token rows of
//               every activation tile (the MMA reads the other half from the peer's shared memory), which halves
//               the activation bytes each SM pulls from L2 per FLOP.  The even-ranked CTA (leader) issues the MMAs;
//               its "full" barriers collect the arrivals and TMA bytes of both CTAs, and its commits release the
//               stages in both.
// XROWS = token rows of an activation stage (256, or 128 in the few-token variant: tokens <= 128, single CTA, the
//         shared memory saved goes to the ring of packed weight blocks).
template <int QT, typename T16, bool BWD, bool PAIR, int MTOK, int XROWS>
__global__ void __launch_bounds__(kThreads, 1) k_umma_gemm(const __grid_constant__ Params p) {
    using QS = QuantStage<QT>;
    constexpr int H = QS::kHdrBytes, Q1 = QS::kQ1Bytes;
    static_assert(XROWS == 256 || XROWS == 128, "activation stage: 256 or 128 token rows per CTA");
    constexpr int kXStageBytes = XROWS * 128;
    constexpr int kOffA = kOffX + kNumA * kXStageBytes;
    constexpr int kOffRaw = kOffA + kNumA * kAStageBytes;
    constexpr int kRawBudget = kOffBar - kOffRaw;
    // fp16 weights: no packed-block ring and no dequantization - the weight producer's TMA copies land in the operand
    // stage itself (128-byte swizzle = the tile image the dequantizer would have written)
    constexpr bool kDirect = QT == kTypeF16;
    constexpr int kRows = BWD ? 64 : 128;      // weight rows per raw stage
    constexpr int kSub = BWD ? 1 : 2;          // operand stages produced per raw stage
    constexpr int kNumX = kNumA;
    constexpr int kRawStageBytes = (kRows * (H + 64 + Q1) + 1023) & ~1023;
    // Ring of packed blocks.  An mbarrier wait names a phase by its parity, so whoever waits on a barrier must visit
    // EVERY phase of it, one after the other (a waiter two phases behind would take the phase before last for the one
    // it wants).  The dequant groups walk the raw stages with stride kStride (forward: two groups share a raw stage, the
    // pairs alternate; backward: the four groups take every fourth stage).  Where kStride does not divide the number
    // of slots, a slot gets one full / empty barrier pair per residue class r % kStride of the stages it holds: a
    // barrier (slot, class) then sees the stages r0, r0 + kLcm, r0 + 2 kLcm, ... and always the same waiters.  The
    // producer teams (stride kTeams, a divisor of kStride) wait for the stage that held the slot before.
    constexpr int kStride = BWD ? 4 : 2;
    constexpr int kFit = kRawBudget / kRawStageBytes;
    constexpr int kNumRaw = kFit < kMaxRaw ? (kFit < 1 ? 1 : kFit) : kMaxRaw;
    constexpr int kCls = kNumRaw % kStride == 0 ? 1 : kStride;
    constexpr int kLcm = kNumRaw % kStride == 0 ? kNumRaw : (kNumRaw % 2 == 0 ? 2 * kNumRaw : kStride * kNumRaw);
    constexpr int kTeams = kStride;      // weight-producer teams (three lanes each)
    static_assert(kDirect || kNumRaw * kCls <= kMaxRawBars, "not enough barrier slots for the raw ring");
    static_assert(kLcm % kNumRaw == 0 && kLcm % kStride == 0, "kLcm is a common multiple");
    // MTOK = token columns per MMA (the accumulator is cut into 512 / MTOK independent tiles that the issuer visits
    // round-robin); kMmaSlotBytes = smem bytes of one MMA's activation rows in a stage
    constexpr int kMmaSlotBytes = (PAIR ? MTOK / 2 : MTOK) * 128;
    constexpr uint32_t kFmt = std::is_same<T16, __half>::value ? 0u : 1u;   // UMMA operand format: 0 f16, 1 bf16

    extern __shared__ uint8_t smem_dyn[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBar;
    auto bar = [&](int slot) -> uint32_t { return bar0 + 8u * (uint32_t)slot; };
    // raw stage r (counted from this CTA's first one): its barrier index inside the full / empty arrays, and its phase
    auto raw_bar = [&](int r) -> int { return (r % kNumRaw) * kCls + (kCls > 1 ? r % kStride : 0); };
    auto raw_phase = [&](int r) -> uint32_t { return (uint32_t)(r / kLcm) & 1u; };
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + kOffBar + kOffAbort);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kOffBar + kOffTmemSlot);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;        // 0 = leader
    const bool leader = crank == 0;
    const int tok0 = blockIdx.z * kMaxTok;
    const int tok_left = p.T - tok0;
    // token columns of this CTA's accumulator: multiple of 16 (single) / 32 (pair, 16 per CTA half)
    const int tb = PAIR ? min(kMaxTok, (tok_left + 31) & ~31) : min(kMaxTok, (tok_left + 15) & ~15);
    const int n_box = (tb + p.t_box - 1) / p.t_box;             // single-CTA mode: TMA boxes per stage
    const int n_mma = (tb + MTOK - 1) / MTOK;
    // Few tokens (single-CTA mode): the four k-steps of a stage go to separate accumulators, so they do not wait on
    // each other's accumulation (a dependent MMA costs ~250 clocks whatever its size); the epilogue adds them up.
    const int acc_stride = (tb + 31) & ~31;
    const int n_acc = n_mma > 1 ? 1 : (acc_stride <= 128 ? 4 : (acc_stride <= 256 ? 2 : 1));
    const int u0 = (int)((int64_t)p.units * split / p.splits);
    const int u1 = (int)((int64_t)p.units * (split + 1) / p.splits);
    // Up to 128 tokens (single-CTA mode) the kernel is bound by how fast MMAs can be ISSUED (an MMA of 16..128 token
    // columns costs its issuing thread about as much as a full-width one): the two issuers then work side by side, each
    // on its own set of partial accumulators (no turn token; every accumulator still receives its MMAs from one thread
    // in a fixed order, so results do not change from run to run).  Needs a main stage for either issuer.
    const bool par = !PAIR && p.par_ok != 0 && acc_stride <= 128 && (u1 - u0) * (BWD ? 1 : 2) >= 2;
    const int n_acc_per = par ? (acc_stride <= 64 ? 4 : 2) : n_acc;      // partial accumulators per issuer
    const int n_acc_sum = par ? 2 * n_acc_per : n_acc;                   // ... that the epilogue adds up
    // forward: the member that owns this tile; backward: every CTA works on all members, unit by unit
    int mi = 0;
    if (!BWD)
        for (int j = 1; j < p.n_members; j++)
            if (tile >= p.m[j].first) mi = j;
    const Member &M = p.m[mi];
    const int ltile = BWD ? tile : tile - M.first;
    // backward: global unit index -> (member, 64-row block inside it)
    auto unit_member = [&](int u, int &rb) -> int {
        int j = 0;
        rb = u;
        while (j + 1 < p.n_members && rb >= p.m[j].count) {
            rb -= p.m[j].count;
            j++;
        }
        return j;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumRaw * kCls; i++) {
            mbar_init(bar(kBarRawFull + i), 1);
            mbar_init(bar(kBarRawEmpty + i), BWD ? 4 : 8);       // one arrival per warp that read the stage
        }
        for (int i = 0; i < kNumA; i++) {
            // full: the (leader's) producer arrival carrying the TMA bytes + one arrival per dequant warp (of both CTAs)
            // (a dequant warp counts four times: one group of 4 warps produces a stage, rank-update stages included)
            // (fp16 weights: the activation producer and the weight producer, one arrival each)
            mbar_init(bar(kBarFull + i), kDirect ? 2 : 1 + (PAIR ? 32 : 16));
            mbar_init(bar(kBarEmpty + i), 1);                    // tcgen05.commit of the stage's MMAs
        }
        mbar_init(bar(kBarAcc), 2);        // both MMA issuers commit to it
        mbar_init(bar(kBarTurn + 0), 1);   // issuer 1 has queued its stage: issuer 0 may queue the next one
        mbar_init(bar(kBarTurn + 1), 1);   // and the other way round (stage order = accumulation order, run to run)
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.m[0].tm_act);
        tma_prefetch_desc(&M.tm_hdr);
        tma_prefetch_desc(&M.tm_q0);
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(sbase + kOffBar + kOffTmemSlot, (uint32_t)p.tmem_cols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(sbase + kOffBar + kOffTmemSlot, (uint32_t)p.tmem_cols);
            tmem_relinquish();
        }
    }
    // Programmatic dependent launch: this CTA may start while the kernel before it in the stream (the pass that wrote
    // the 16-bit activations, the low-rank activations and the output's bias / zero fill) still runs; every kernel
    // before THAT one has completed, because it passed its own wait before it let this one be scheduled.  The packed
    // weights, the adapter matrices and the adapter's non-zero flag are not written by that pass, so the weight producer
    // and the dequant warps start at once and the first operand stages are ready when the activations arrive; whoever
    // touches what the pass wrote waits for it first: the activation producer before its first copy, the dequant warps
    // before the rank-update stage and the epilogue.  The next kernel may be scheduled behind this one right away.
    pdl_trigger();
    // rank-update stages (split 0 only): forward one for this tile's member, backward one per member with an adapter
    int lora_m[kMaxMembers];
    int n_lora = 0;
    int dual_pad[2] = {0, 0};      // dual forward: 16-padded ranks of the two members inside the one rank-update stage
    if (split == 0) {
        if (!BWD && p.dual) {
            for (int j = 0; j < 2; j++)
                if (p.m[j].rank > 0 && (p.m[j].lora_flag == nullptr || *p.m[j].lora_flag != 0)) dual_pad[j] = (p.m[j].rank + 15) & ~15;
            if (dual_pad[0] + dual_pad[1] > 0) lora_m[n_lora++] = 0;
        } else if (!BWD) {
            if (M.rank > 0 && (M.lora_flag == nullptr || *M.lora_flag != 0)) lora_m[n_lora++] = mi;
        } else {
            for (int j = 0; j < p.n_members; j++)
                if (p.m[j].rank > 0) lora_m[n_lora++] = j;
        }
    }
    tc_fence_before_sync();
    if (PAIR) cluster_sync_all(); else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    auto trace = [&](int row, int idx) {
        if (tracing && idx < 128) p.trace[row * 128 + idx] = clock64();
    };
    if (threadIdx.x == 0) trace(11, 0);
    if (p.trace != nullptr && threadIdx.x == 0) {       // wall-clock span of the grid: latest start / end over all CTAs
        const unsigned long long now = globaltimer_ns();
        if (tracing) p.trace[11 * 128 + 8] = (long long)now;
        atomicMax(reinterpret_cast<unsigned long long *>(p.trace) + 11 * 128 + 10, (1ull << 62) - now);
    }

    // activation tile of one stage: coordinate c0 along the contraction, this CTA's token rows
    // Called by lanes 0..3 of the activation producer warp: lane 0 arms the barrier, lane i issues copy i (the copies
    // of a stage are issued side by side; the barrier cannot complete before lane 0's arrival).
    auto load_act_stage = [&](const CUtensorMap *tm, int c0, uint32_t xdst, uint32_t xbar_local, int li) {
        if (PAIR) {
            // leader arms the barrier for the bytes of both CTAs; each CTA loads its half of every MMA's tokens
            if (leader && li == 0) mbar_arrive_expect_tx(xbar_local, (uint32_t)(2 * n_mma * (MTOK / 2) * 128));
            const uint32_t lbar = mapa_cluster(xbar_local, 0);
            if (li < n_mma) {
                const int ntok = min(MTOK, tb - MTOK * li);
                tma_load_2d_pair(xdst + li * kMmaSlotBytes, tm, c0, tok0 + MTOK * li + (int)crank * (ntok >> 1), lbar);
            }
        } else {
            if (li == 0) mbar_arrive_expect_tx(xbar_local, (uint32_t)(n_box * p.t_box * 128));
            if (li < n_box) tma_load_2d(xdst + li * p.t_box * 128, tm, c0, tok0 + li * p.t_box, xbar_local);
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer of the packed weights
        // (issuing a tiled copy costs the issuing thread several hundred clocks: weights and activations have a
        // producer thread each, on their own barriers)
        if (kDirect) {
            // fp16 rows: lane 0 waits for the operand stage, arms the (leader's) full barrier for the bytes of both
            // CTAs and copies this CTA's 128 rows x 64 columns; backward: lanes 0 and 1 copy the two 64-column images
            if (lane < (BWD ? 2 : 1)) {
                Ring as;
                bool ok = true;
                for (int u = u0; u < u1 && ok; u++) {
                    int um = mi, rb = 0;
                    if (BWD) um = unit_member(u, rb);
                    const Member &W = p.m[um];
                    for (int s = 0; s < kSub && ok; s++) {
                        ok = mbar_wait_bounded(bar(kBarEmpty + as.idx), as.phase ^ 1u, abort_flag, p.status, kCodeProducer + 1);
                        if (!ok) break;
                        const uint32_t adst = sbase + kOffA + as.idx * kAStageBytes;
                        const uint32_t fbar_local = bar(kBarFull + as.idx);
                        const uint32_t fbar = PAIR ? mapa_cluster(fbar_local, 0) : fbar_local;
                        if (lane == 0 && leader) mbar_arrive_expect_tx(fbar_local, (uint32_t)((PAIR ? 2 : 1) * kAStageBytes));
                        if (BWD) {
                            // image `lane`: weight rows rb*64.., columns tile*128 + 64*lane ..
                            const int x = (tile * kTileW + 64 * lane) * 2, y = W.row_base + rb * 64;
                            if (PAIR) tma_load_2d_pair(adst + lane * 8192, &W.tm_q0, x, y, fbar);
                            else tma_load_2d(adst + lane * 8192, &W.tm_q0, x, y, fbar);
                        } else {
                            const int x = (u * 2 + s) * 64 * 2, y = W.row_base + ltile * kTileW;
                            if (PAIR) tma_load_2d_pair(adst, &W.tm_q0, x, y, fbar);
                            else tma_load_2d(adst, &W.tm_q0, x, y, fbar);
                        }
                        if (lane == 0) trace(0, (u - u0) * kSub + s);
                        as.advance(kNumA);
                    }
                }
            }
        } else if (lane < ((!BWD && p.dual) ? 6 : 3) * kTeams) {
            // Teams of three lanes (lane 0 of a team arms the barrier and copies the headers, lanes 1 and 2 copy the
            // quant regions); team t issues the raw stages r = t (mod kTeams).  Issuing a tiled copy holds the issuing
            // thread for several hundred clocks: with one team the issue rate alone (one raw stage per ~800 clocks) paced
            // the few-token shapes.  kTeams <= kNumRaw, so a team never waits for a slot whose previous stage is issued
            // in the same round.
            // (dual forward: six lanes, one per region and member)
            const int lpt = (!BWD && p.dual) ? 6 : 3;
            const int team = lane / lpt, li = lane - lpt * team;
            bool ok = true;
            for (int u = u0 + team; u < u1 && ok; u += kTeams) {
                const int r = u - u0, ri = r % kNumRaw;
                // the slot's previous stage has been read
                if (r >= kNumRaw)
                    ok = mbar_wait_bounded(bar(kBarRawEmpty + raw_bar(r - kNumRaw)), raw_phase(r - kNumRaw), abort_flag, p.status, kCodeProducer + 1);
                if (!ok) break;
                const uint32_t rdst = sbase + kOffRaw + ri * kRawStageBytes;
                const uint32_t rbar = bar(kBarRawFull + raw_bar(r));
                int sb, half, row0, um = mi, rb = 0;
                if (BWD) {
                    um = unit_member(u, rb);
                    sb = tile >> 1; half = tile & 1; row0 = rb * 64;
                } else {
                    sb = u >> 1; half = u & 1; row0 = ltile * kTileW;
                }
                const Member &W = p.m[um];
                row0 += W.row_base;
                const int xb = sb * QS::kBlockBytes;
                if (!BWD && p.dual) {
                    // 64 rows of either member (64-row boxes): member 1's rows land behind member 0's in every region
                    const int reg = li % 3, mm = li / 3;
                    const int region = reg == 0 ? 0 : (reg == 1 ? kRows * H : kRows * (H + 64));
                    const int row_bytes = reg == 0 ? H : (reg == 1 ? 64 : Q1);
                    const int x = xb + (reg == 0 ? QS::hdr_x(half) : (reg == 1 ? QS::q0_x(half) : QS::q1_x(half)));
                    if (li == 0) {
                        mbar_arrive_expect_tx(rbar, (uint32_t)(kRows * (H + 64 + Q1)));
                        if (lane == 0) trace(0, r / kTeams);
                    }
                    if (reg < 2 || Q1 > 0) {
                        const Member &Wm = p.m[mm];
                        const CUtensorMap *tm = reg == 0 ? &Wm.tm_hdr : (reg == 1 ? &Wm.tm_q0 : &Wm.tm_q1);
                        tma_load_2d(rdst + region + mm * 64 * row_bytes, tm, x, Wm.row_base + ltile * 64, rbar);
                    }
                    continue;
                }
                // one copy per region: the tensor maps handed to a forward launch have 128-row boxes, the backward
                // ones 64-row boxes
                if (li == 0) {
                    mbar_arrive_expect_tx(rbar, (uint32_t)(kRows * (H + 64 + Q1)));
                    tma_load_2d(rdst, &W.tm_hdr, xb + QS::hdr_x(half), row0, rbar);
                    if (lane == 0) trace(0, r / kTeams);
                } else if (li == 1) {
                    tma_load_2d(rdst + kRows * H, &W.tm_q0, xb + QS::q0_x(half), row0, rbar);
                } else if (Q1 > 0) {
                    tma_load_2d(rdst + kRows * (H + 64), &W.tm_q1, xb + QS::q1_x(half), row0, rbar);
                }
            }
        }
    } else if (warp == kActProducerWarp) {
        // ------------------------------------------------------------------ TMA producer of the activation tiles
        if (lane < 4) {
            Ring xs;
            bool ok = true;
            pdl_wait();      // the activations come from the kernel before this one
            for (int u = u0; u < u1 && ok; u++) {
                int um = mi, rb = 0;
                if (BWD) um = unit_member(u, rb);
                const Member &W = p.m[um];
                for (int s = 0; s < kSub && ok; s++) {
                    ok = mbar_wait_bounded(bar(kBarEmpty + xs.idx), xs.phase ^ 1u, abort_flag, p.status, kCodeProducer + 2);
                    if (!ok) break;
                    load_act_stage(BWD ? &W.tm_act : &p.m[0].tm_act, BWD ? rb * 64 : (u * 2 + s) * 64, sbase + kOffX + xs.idx * kXStageBytes,
                                   bar(kBarFull + xs.idx), lane);
                    if (lane == 0) trace(1, (u - u0) * kSub + s);
                    xs.advance(kNumX);
                }
            }
            for (int j = 0; j < n_lora && ok; j++) {
                // rank-update stage: both operand tiles are built by the dequant warps; the producer only adds the
                // arrival that stands for the TMA bytes in the other stages
                ok = mbar_wait_bounded(bar(kBarEmpty + xs.idx), xs.phase ^ 1u, abort_flag, p.status, kCodeProducer + 3);
                if (ok && leader && lane == 0) mbar_arrive(bar(kBarFull + xs.idx));
                xs.advance(kNumX);
            }
        }
    } else if (warp == 1 || warp == kIssuer2Warp) {
        // ------------------------------------------------------------------ two MMA issuers (leader CTA only in pair mode)
        // Issuing is blocking (the queue in front of the tensor pipe is short) and every stage costs a barrier wait,
        // a fence and a commit: two threads take alternate stages, so one waits for its next stage while the other
        // keeps the pipe fed.  They hand a turn token back and forth, so stages are queued in order and the fp32
        // accumulation order does not change from run to run.  tcgen05.commit tracks the MMAs of the committing thread, so each releases its own stages.
        if (lane == 0 && leader) {
            const int who = warp == 1 ? 0 : 1;
            bool ok = true;
            const uint32_t a_mn = BWD ? 1u : 0u;
            auto wait_full = [&](int n, int code) -> bool {
                const int slot = kBarFull + (n % kNumA);
                const uint32_t phase = (uint32_t)(n / kNumA) & 1u;
                const bool r = PAIR ? mbar_wait_bounded_cluster(bar(slot), phase, abort_flag, p.status, code)
                                    : mbar_wait_bounded(bar(slot), phase, abort_flag, p.status, code);
                tc_fence_after_sync();
                return r;
            };
            const int n_main = (u1 - u0) * kSub;
            const int n_total = n_main + n_lora;
            // Everything an MMA needs is precomputed: the issuing thread is one thread, and at ~5 clocks per dependent
            // instruction a few dozen instructions per MMA would cost more than the MMA itself.
            // descriptor = (lo, hi): lo = (addr >> 4) | (LBO >> 4) << 16, hi = (SBO >> 4) | version 1 << 14 | SWIZZLE_128B << 29
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t kALoField = (BWD ? (8192u >> 4) : 1u) << 16;     // MN-major: LBO = stride between 64-column images
            constexpr uint32_t kAStep = (BWD ? 2048u : 32u) >> 4;               // per k-step advance of the A operand
            constexpr int kMaxMma = 512 / MTOK;
            uint32_t idesc[kMaxMma];
#pragma unroll
            for (int i = 0; i < kMaxMma; i++) {
                const int ntok = max(16, min(MTOK, tb - MTOK * i));
                idesc[i] = umma_idesc_f16(kFmt, a_mn, 0u, (uint32_t)ntok, PAIR ? 256u : 128u);
            }
            for (int n = who; n < n_total && ok; n += 2) {
                ok = wait_full(n, kCodeMma + 1);
                if (!ok) break;
                const int si = n % kNumA;
                const uint32_t a_lo0 = (((sbase + kOffA + si * kAStageBytes) & 0x3FFFFu) >> 4) | kALoField;
                const uint32_t b_lo0 = (((sbase + kOffX + si * kXStageBytes) & 0x3FFFFu) >> 4) | (1u << 16);
                const int ksteps = n < n_main ? 4 : ((!BWD && p.dual) ? (dual_pad[0] + dual_pad[1]) >> 4 : ((p.m[lora_m[n - n_main]].rank + 15) >> 4));
                if (n > 0 && !par) {
                    // take the turn: the other issuer has queued stage n - 1 (by now this thread has already waited for
                    // its own operands, which is the latency the second issuer hides)
                    const uint32_t turn_phase = (uint32_t)(who == 1 ? (n >> 1) : ((n >> 1) - 1)) & 1u;
                    ok = mbar_wait_bounded(bar(kBarTurn + who), turn_phase, abort_flag, p.status, kCodeMma + 5);
                    if (!ok) break;
                }
                if (who == 0) trace(8, n);
                const uint32_t first = n == (par ? who : 0) ? 0u : 1u;     // the very first MMA into an accumulator overwrites it
                // k-step-major order: consecutive MMAs alternate between the accumulators (measured faster than
                // finishing one accumulator's k-steps first)
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    if (ks < ksteps) {
                        const uint32_t a_lo = a_lo0 + ks * kAStep;
                        if (PAIR && n_mma > 1) {
#pragma unroll
                            for (int i = 0; i < kMaxMma; i++)
                                if (i < n_mma)
                                    umma_f16_ss_lohi<true>(tmem_base + i * MTOK, a_lo, kDescHi, b_lo0 + i * (kMmaSlotBytes >> 4) + ks * 2,
                                                           kDescHi, idesc[i], ks == 0 ? first : 1u);
                        } else if (PAIR) {
                            // one MMA per k-step (tokens <= MTOK): each k-step into its own partial accumulator
                            const int a = ks % n_acc;
                            umma_f16_ss_lohi<true>(tmem_base + a * acc_stride, a_lo, kDescHi, b_lo0 + ks * 2, kDescHi, idesc[0],
                                                   ks < n_acc ? first : 1u);
                        } else {
                            // few tokens: one MMA per k-step, each k-step into its own partial accumulator
                            const int a = (par ? who * n_acc_per : 0) + ks % n_acc_per;
                            umma_f16_ss_lohi<false>(tmem_base + a * acc_stride, a_lo, kDescHi, b_lo0 + ks * 2, kDescHi, idesc[0],
                                                    ks < n_acc_per ? first : 1u);
                        }
                    }
                }
                if (PAIR) umma_commit_pair(bar(kBarEmpty + si)); else umma_commit(bar(kBarEmpty + si));
                if (!par) mbar_arrive(bar(kBarTurn + (who ^ 1)));
                if (who == 0) trace(9, n);
            }
            if (ok) {
                if (PAIR) umma_commit_pair(bar(kBarAcc)); else umma_commit(bar(kBarAcc));
            }
        }
    } else {
        // ------------------------------------------------------------------ dequant warps, then epilogue
        // Four groups of four warps; group g4 produces the operand stages n = g4 (mod 4), always into A slot g4, so
        // four stages are being dequantized at any time (one stage is a chain of waits, shared-memory round trips and
        // a proxy fence, about a thousand clocks whatever the number of threads working on it: the groups hide each
        // other's latency).  A thread produces 64 weights of a stage as two independent 32-weight runs.
        const int dt = (threadIdx.x - 64) & 127;        // thread index inside its 4-warp group
        const int g4 = (warp - 2) >> 2;                 // group 0..3
        const int nu = u1 - u0;
        bool ok = true;
        // "operand stage ready": on the barrier of the CTA that issues the MMAs
        auto signal_a_full = [&](int ai, uint32_t count) {
            if (lane == 0) {
                if (PAIR && !leader) mbar_arrive_cluster_n(mapa_cluster(bar(kBarFull + ai), 0), count);
                else mbar_arrive_n(bar(kBarFull + ai), count);
            }
        };
        // operand stage n lives in A slot n % kNumA with phase (n / kNumA) & 1; raw stage i in slot i % kNumRaw.
        // Runs r = 0, 1 of this thread: 32-weight group grp[r] of the row, written at dst_off[r] + chunk0[r].
        auto produce = [&](int n, const uint8_t *rs, int row, int half, const int (&grp)[2], const uint32_t (&dst_off)[2],
                           const int (&chunk0)[2]) -> bool {
            const int ai = n % kNumA;
            if (!mbar_wait_bounded(bar(kBarEmpty + ai), ((uint32_t)(n / kNumA) & 1u) ^ 1u, abort_flag, p.status, kCodeDequant + 2))
                return false;
            if (dt == 0 && g4 < 2) trace(3 + 3 * g4, n);
            const uint32_t a_addr = sbase + kOffA + ai * kAStageBytes;
#pragma unroll
            for (int r = 0; r < 2; r++)
                dequant32_to_swizzled_row<QT, T16>(rs + row * H, rs + kRows * H + row * 64,
                                                   rs + kRows * (H + 64) + row * (Q1 > 0 ? Q1 : 1), (row >> 1) & 3, (row >> 2) & 1,
                                                   half, grp[r], a_addr + dst_off[r], row & 7, chunk0[r]);
            fence_proxy_async_smem();
            __syncwarp();
            signal_a_full(ai, 4);
            if (dt == 0 && g4 < 2) trace(4 + 3 * g4, n);
            return true;
        };
        if (kDirect) {
            // nothing to dequantize
        } else if (!BWD) {
            // raw stage = 128 rows x half block = two operand stages (its 64-column halves); groups 0, 1 take the even
            // raw stages, groups 2, 3 the odd ones; a thread owns one row of its group's half
            const int row = dt, sub = g4 & 1;
            const int grp[2] = {2 * sub, 2 * sub + 1};
            const int prow = p.dual ? dual_row(row) : row;      // (prow & 7 == row & 7: the swizzle phase stays the row's)
            const uint32_t dst_off[2] = {(uint32_t)(prow * 128), (uint32_t)(prow * 128)};
            const int chunk0[2] = {0, 4};
            for (int ui = g4 >> 1; ui < nu && ok; ui += 2) {
                const int ri = ui % kNumRaw;
                ok = mbar_wait_bounded(bar(kBarRawFull + raw_bar(ui)), raw_phase(ui), abort_flag, p.status, kCodeDequant + 1);
                if (!ok) break;
                if (dt == 0 && g4 < 2) trace(2 + 3 * g4, 2 * ui + sub);
                const uint8_t *rs = smem + kOffRaw + ri * kRawStageBytes;
                ok = produce(2 * ui + sub, rs, row, (u0 + ui) & 1, grp, dst_off, chunk0);
                if (!ok) break;
                if (lane == 0) mbar_arrive(bar(kBarRawEmpty + raw_bar(ui)));
            }
        } else {
            // raw stage = 64 rows x half block = one operand stage (two 64-column images); group g4 takes the stages
            // ui = g4 (mod 4); a thread owns one row of one image
            const int row = dt & 63, im = dt >> 6;
            const int grp[2] = {2 * im, 2 * im + 1};
            const uint32_t dst_off[2] = {(uint32_t)(im * 8192 + row * 128), (uint32_t)(im * 8192 + row * 128)};
            const int chunk0[2] = {0, 4};
            for (int ui = g4; ui < nu && ok; ui += 4) {
                const int ri = ui % kNumRaw;
                ok = mbar_wait_bounded(bar(kBarRawFull + raw_bar(ui)), raw_phase(ui), abort_flag, p.status, kCodeDequant + 1);
                if (!ok) break;
                if (dt == 0 && g4 < 2) trace(2 + 3 * g4, ui);
                const uint8_t *rs = smem + kOffRaw + ri * kRawStageBytes;
                ok = produce(ui, rs, row, tile & 1, grp, dst_off, chunk0);
                if (!ok) break;
                if (lane == 0) mbar_arrive(bar(kBarRawEmpty + raw_bar(ui)));
            }
        }
        pdl_wait();      // from here on: the low-rank activations, the bias, the output
        // A rank-update stage is built by the group that owns its slot (n % 4), like any other stage of that slot: the
        // group has seen every phase of the slot's barriers.  (A group that never waited on a slot could take a phase
        // two behind for the one it wants - parity waits cannot tell them apart - and the two MMA issuers may be many
        // stages apart when they run side by side.)
        for (int lj = 0; lj < n_lora && ok; lj++) {
            // weight-side tile from B (forward) / A (backward), activation-side tile from the fp32 low-rank activations,
            // both rounded to T16 here
            const Member &L = p.m[lora_m[lj]];
            const int rank_pad = (!BWD && p.dual) ? dual_pad[0] + dual_pad[1] : (L.rank + 15) & ~15;
            const int n = (BWD ? 1 : 2) * nu + lj;
            const int ai = n % kNumA;
            if (ai != g4) continue;
            ok = mbar_wait_bounded(bar(kBarEmpty + ai), ((uint32_t)(n / kNumA) & 1u) ^ 1u, abort_flag, p.status, kCodeDequant + 3);
            if (!ok) break;
            const uint32_t a_addr = sbase + kOffA + ai * kAStageBytes;
            if (!BWD && p.dual) {
                // one stage for both members: contraction columns [0, pad0) are member 0's ranks, [pad0, pad0 + pad1) member
                // 1's; a member's weight-side rows are zero in the other member's columns
                const uint32_t x_addr = sbase + kOffX + ai * kXStageBytes;
                for (int i = 0; i < n_mma; i++) {
                    const int ntok = min(MTOK, tb - MTOK * i);
                    const int rows = PAIR ? (ntok >> 1) : ntok;
                    for (int rr = dt; rr < rows; rr += 128) {
                        const int t = tok0 + MTOK * i + (PAIR ? (int)crank * rows : 0) + rr;
                        const uint32_t row_addr = x_addr + (uint32_t)(i * kMmaSlotBytes + rr * 128);
                        for (int j = 0; j * 8 < rank_pad; j++) {
                            const int mm = 8 * j < dual_pad[0] ? 0 : 1;
                            const Member &Lm = p.m[mm];
                            const int rbase = 8 * j - (mm ? dual_pad[0] : 0);
                            float v[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                const int r = rbase + q;
                                v[q] = (r < Lm.rank && t < p.T) ? Lm.lora_act[(int64_t)t * Lm.rank + r] * Lm.lora_scale : 0.f;
                            }
                            st_shared_v4(row_addr + (uint32_t)((j ^ (rr & 7)) << 4), pack2<T16>(v[0], v[1]), pack2<T16>(v[2], v[3]),
                                         pack2<T16>(v[4], v[5]), pack2<T16>(v[6], v[7]));
                        }
                    }
                }
                {
                    const int row = dt, mm = row >> 6, nn = ltile * 64 + (row & 63), prow = dual_row(row);
                    const Member &Lm = p.m[mm];
                    for (int j = 0; j * 8 < rank_pad; j++) {
                        const bool mine = (8 * j < dual_pad[0]) == (mm == 0) && dual_pad[mm] > 0;
                        const int rbase = 8 * j - (mm ? dual_pad[0] : 0);
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const int r = rbase + i;
                            v[i] = (mine && r < Lm.rank && nn < Lm.N) ? Lm.lora_w[(int64_t)r * Lm.N + nn] : 0.f;
                        }
                        st_shared_v4(a_addr + (uint32_t)(prow * 128 + ((j ^ (prow & 7)) << 4)), pack2<T16>(v[0], v[1]),
                                     pack2<T16>(v[2], v[3]), pack2<T16>(v[4], v[5]), pack2<T16>(v[6], v[7]));
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                signal_a_full(ai, 4);
                continue;
            }
            {
                // token rows of this CTA's activation tile: rank_pad/8 chunks of a 128-byte row
                const uint32_t x_addr = sbase + kOffX + ai * kXStageBytes;
                for (int i = 0; i < n_mma; i++) {
                    const int ntok = min(MTOK, tb - MTOK * i);
                    const int rows = PAIR ? (ntok >> 1) : ntok;
                    for (int rr = dt; rr < rows; rr += 128) {
                        const int t = tok0 + MTOK * i + (PAIR ? (int)crank * rows : 0) + rr;
                        const uint32_t row_addr = x_addr + (uint32_t)(i * kMmaSlotBytes + rr * 128);
                        for (int j = 0; j * 8 < rank_pad; j++) {
                            float v[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                const int r = 8 * j + q;
                                v[q] = (r < L.rank && t < p.T) ? L.lora_act[(int64_t)t * L.rank + r] * L.lora_scale : 0.f;
                            }
                            st_shared_v4(row_addr + (uint32_t)((j ^ (rr & 7)) << 4), pack2<T16>(v[0], v[1]), pack2<T16>(v[2], v[3]),
                                         pack2<T16>(v[4], v[5]), pack2<T16>(v[6], v[7]));
                        }
                    }
                }
            }
            if (!BWD) {
                // image[row = n][col = r] = B[r, n]; chunks of 8 ranks
                const int row = dt, nn = ltile * kTileW + row;
                for (int j = 0; j * 8 < rank_pad; j++) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int r = 8 * j + i;
                        v[i] = (r < L.rank && nn < L.N) ? L.lora_w[(int64_t)r * L.N + nn] : 0.f;
                    }
                    st_shared_v4(a_addr + (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4)), pack2<T16>(v[0], v[1]),
                                 pack2<T16>(v[2], v[3]), pack2<T16>(v[4], v[5]), pack2<T16>(v[6], v[7]));
                }
            } else {
                // image(kcol >> 6)[row = r][col = kcol & 63] = A[k, r]
                const int kcol = dt, c = kcol & 63, k = tile * kTileW + kcol;
                for (int r = 0; r < rank_pad; r++) {
                    const float v = (r < L.rank && k < p.K) ? L.lora_w[(int64_t)k * L.rank + r] : 0.f;
                    const uint32_t addr =
                        a_addr + (uint32_t)((kcol >> 6) * 8192 + r * 128 + (((c >> 3) ^ (r & 7)) << 4) + (c & 7) * 2);
                    const uint32_t bits = pack2<T16>(v, 0.f) & 0xFFFFu;
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)bits) : "memory");
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            signal_a_full(ai, 4);
        }
        // epilogue: TMEM lane = weight row / column of this tile, TMEM column = token
        if (ok) ok = mbar_wait_bounded(bar(kBarAcc), 0u, abort_flag, p.status, kCodeEpilogue + 1, 16000000000ll);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-collective: take the epilogue only as a whole warp
        if (!BWD && p.dual) {
            // the dual epilogue's warps meet at named barriers: all sixteen take it, or none (a warp whose wait gave up has
            // raised the CTA's abort flag)
            asm volatile("bar.sync 5, 512;" ::: "memory");
            ok = *abort_flag == 0;
        }
        if (ok) {
            tc_fence_after_sync();
            if (threadIdx.x == 64) trace(11, 1);
            const int quad = warp & 3, cgrp = (warp - 2) >> 2;     // TMEM lane quadrant; column group 0..3
            if (!BWD && p.dual) {
                // Lanes 0..15 of the warp hold member 0 (gate), lanes 16..31 member 1 (up) of the same 16 features.  The four
                // warps of a column group stage their 32 tokens x 64 features in shared memory (the operand stages are free:
                // every MMA has completed) and write them out a whole row of the tile per instruction - 128 bytes of the
                // 16-bit product, 256 of gate or up; straight from the registers a warp would write 32- and 64-byte pieces,
                // and the drain of the tile is bound by the number of requests, not by their bytes.  Shared memory is
                // addressed by 32-bit offsets with immediate displacements: the loops below are bound by instruction issue.
                const int mm = lane >> 4;
                const int fcol = quad * 16 + (lane & 15);
                const int f0 = ltile * 64;
                const Member &Mm = p.m[mm];
                const bool tile_ok = f0 < Mm.N;      // out_features % 64 == 0: a tile is all in range or (pair padding) all out
                const float bvm = (Mm.bias && tile_ok) ? Mm.bias[f0 + fcol] : 0.f;
                float *const out_g = p.m[0].out, *const out_u = p.m[1].out;
                const bool stage_gu = out_g != nullptr || out_u != nullptr;
                const int ld_gu = p.m[0].ld_out;
                T16 *const h16 = reinterpret_cast<T16 *>(p.h16);
                // staging of this column group: [32][64] 16-bit product | [32][64] fp32 gate | [32][64] fp32 up
                const uint32_t stg = sbase + kOffX + (uint32_t)cgrp * 20480u;
                const uint32_t st_x = stg + (mm ? 12288u : 4096u) + (uint32_t)fcol * 4u;      // this lane's member, row j
                const uint32_t st_h = stg + (uint32_t)(mm * 64 + fcol) * 2u;                  // product of token j + mm
                const uint32_t ld_h = stg + (uint32_t)(quad * 8) * 128u + (uint32_t)lane * 4u;
                const uint32_t ld_g = stg + 4096u + (uint32_t)(quad * 8) * 256u + (uint32_t)lane * 8u;
                const int nchd = (tb + 31) >> 5;
                const int tok_lim = min(tb, p.T - tok0);      // token rows of this CTA that exist
                for (int c = cgrp; c < nchd; c += 4) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    for (int a = 1; a < n_acc_sum; a++) {
                        uint32_t w2[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * acc_stride + c * 32), w2);
                        tmem_ld_wait();
#pragma unroll
                        for (int jx = 0; jx < 32; jx++) v[jx] = __float_as_uint(__uint_as_float(v[jx]) + __uint_as_float(w2[jx]));
                    }
                    // SiLU(gate) * up (SwiGluKernel.cs:13-35), two tokens per step: the gate lanes take token j (up comes from
                    // the partner lane), the up lanes token j + 1 (gate comes from the partner).  ex2 / rcp approximations:
                    // the product is rounded to 16 bits right here.
#pragma unroll
                    for (int jx = 0; jx < 32; jx += 2) {
                        const float x0 = __uint_as_float(v[jx]) + bvm, x1 = __uint_as_float(v[jx + 1]) + bvm;
                        if (stage_gu) {
                            asm volatile("st.shared.f32 [%0], %1;" ::"r"(st_x + jx * 256), "f"(x0) : "memory");
                            asm volatile("st.shared.f32 [%0], %1;" ::"r"(st_x + (jx + 1) * 256), "f"(x1) : "memory");
                        }
                        const float other = __shfl_xor_sync(0xffffffffu, mm ? x0 : x1, 16);
                        const float g = mm ? other : x0, u = mm ? x1 : other;
                        float sig;
                        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sig) : "f"(1.0f + __expf(-g)));
                        const T16 hv = T16(g * sig * u);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(st_h + jx * 128), "h"(*reinterpret_cast<const unsigned short *>(&hv)) : "memory");
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + cgrp) : "memory");
                    // this warp writes token rows quad * 8 .. + 7 of the chunk
                    const int row0 = c * 32 + quad * 8;
                    const int n_rows = tile_ok ? max(0, min(8, tok_lim - row0)) : 0;
                    const int64_t t_first = (int64_t)tok0 + row0;
                    if (h16 && n_rows > 0) {
                        uint32_t r[8];
#pragma unroll
                        for (int jj = 0; jj < 8; jj++) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[jj]) : "r"(ld_h + jj * 128));
                        T16 *hp = h16 + t_first * p.ld_h16 + f0 + 2 * lane;
#pragma unroll
                        for (int jj = 0; jj < 8; jj++)
                            if (jj < n_rows) *reinterpret_cast<uint32_t *>(hp + (int64_t)jj * p.ld_h16) = r[jj];
                    }
                    if (stage_gu && n_rows > 0) {
#pragma unroll
                        for (int half = 0; half < 2; half++) {
                            float *const op = half ? out_u : out_g;
                            if (!op) continue;
                            float2 r[8];
#pragma unroll
                            for (int jj = 0; jj < 8; jj++)
                                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(r[jj].x), "=f"(r[jj].y) : "r"(ld_g + half * 8192 + jj * 256));
                            float *gp = op + t_first * ld_gu + f0 + 2 * lane;
#pragma unroll
                            for (int jj = 0; jj < 8; jj++)
                                if (jj < n_rows) *reinterpret_cast<float2 *>(gp + (int64_t)jj * ld_gu) = r[jj];
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + cgrp) : "memory");      // the staging tiles are rewritten next
                }
            }
            const int orow = ltile * kTileW + quad * 32 + lane;
            const bool row_ok = orow < (BWD ? p.K : M.N) && !(!BWD && p.dual);
            const float bv = (!BWD && !p.atomic_out && M.bias && row_ok) ? M.bias[orow] : 0.f;
            float *const out_base = M.out;       // backward: member 0 holds the shared dX
            const int ld_out = M.ld_out;
            const int nch = (!BWD && p.dual) ? 0 : (tb + 31) >> 5;      // (the dual forward has written its tile above)
            for (int c = cgrp; c < nch; c += 4) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
                tmem_ld_wait();
                for (int a = 1; a < n_acc_sum; a++) {      // partial accumulators of the few-token mode
                    uint32_t w2[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * acc_stride + c * 32), w2);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w2[j]));
                }
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tl = c * 32 + j;
                        const int t = tok0 + tl;
                        if (tl < tb && t < p.T) {
                            float *dst = out_base + (int64_t)t * ld_out + orow;
                            const float val = __uint_as_float(v[j]);
                            if (p.atomic_out) atomicAdd(dst, val);
                            else *dst = val + bv;       // this CTA alone owns the tile (backward: bv is 0)
                        }
                    }
                }
            }
        }
    }

    if (threadIdx.x == 64) trace(11, 2);
    if (p.trace != nullptr && threadIdx.x == 64) {
        const unsigned long long now = globaltimer_ns();
        if (tracing) p.trace[11 * 128 + 9] = (long long)now;
        atomicMax(reinterpret_cast<unsigned long long *>(p.trace) + 11 * 128 + 11, now);
    }
    if (*abort_flag) {
        // give loads that were already issued time to land before the CTA's shared memory is released
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    // pair mode: neither CTA may leave while the peer's MMAs can still read its shared memory or signal its barriers
    if (PAIR) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        __syncwarp();
        if (PAIR) tmem_dealloc_pair(tmem_base, (uint32_t)p.tmem_cols);
        else tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// A wait that nothing will ever satisfy, with a short limit: exercises the give-up path of mbar_wait_bounded (status
// word written, flag raised, kernel returns normally) without hanging or faulting the device.
__global__ void k_bounded_wait_selftest(int *status, long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar_mem;
    __shared__ int abort_flag;
    const uint32_t b = smem_u32(&bar_mem);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) (void)mbar_wait_bounded(b, 0u, &abort_flag, status, 999, limit_cycles);
    __syncthreads();
    if (threadIdx.x == 1 && abort_flag) atomicAdd(status + 1, 1);     // the other threads saw the flag
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    // function-local static with an initialiser: looked up once, safely from any number of threads
    static const EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

bool encode_2d(CUtensorMap *tm, CUtensorMapDataType dt, int esize, const void *base, uint64_t d0, uint64_t d1,
               uint64_t stride1_bytes, uint32_t b0, uint32_t b1, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t gdim[2] = {d0, d1};
    cuuint64_t gstr[1] = {stride1_bytes};
    cuuint32_t box[2] = {b0, b1};
    cuuint32_t estr[2] = {1, 1};
    (void)esize;
    return fn(tm, dt, 2, const_cast<void *>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int QT, typename T16, bool BWD, bool PAIR, int MTOK, int XROWS>
cudaError_t launch_variant(const Params &p, dim3 grid, cudaStream_t s) {
    static PerDeviceOnce configured;      // one per kernel instantiation
    auto kern = k_umma_gemm<QT, T16, BWD, PAIR, MTOK, XROWS>;
    cudaError_t ce = per_device_once(configured, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes); });
    if (ce != cudaSuccess) return ce;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (PAIR) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 2;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int QT, typename T16, bool BWD>
cudaError_t launch_one(const Params &p, dim3 grid, bool pair, cudaStream_t s) {
    // few tokens: the deep ring of packed blocks (fp16 rows have no packed ring)
    static const bool deep = !(getenv("GT_DEEP_RING") && atoi(getenv("GT_DEEP_RING")) == 0);
    if (pair) {
        if (p.t_box == 64) return launch_variant<QT, T16, BWD, true, 128, 256>(p, grid, s);
        if (QT != kTypeF16 && deep && p.T <= 256) return launch_variant<QT, T16, BWD, true, 256, 128>(p, grid, s);
        return launch_variant<QT, T16, BWD, true, 256, 256>(p, grid, s);
    }
    if (QT != kTypeF16 && deep && p.T <= 128) return launch_variant<QT, T16, BWD, false, 256, 128>(p, grid, s);
    return launch_variant<QT, T16, BWD, false, 256, 256>(p, grid, s);
}

}  // namespace

bool umma_available() { return get_encode_fn() != nullptr; }

bool tmap_encode_2d(CUtensorMap *tm, CUtensorMapDataType dt, const void *base, uint64_t d0, uint64_t d1, uint64_t stride1_bytes,
                    uint32_t b0, uint32_t b1, CUtensorMapSwizzle swz) {
    return encode_2d(tm, dt, 0, base, d0, d1, stride1_bytes, b0, b1, swz);
}

cudaError_t launch_bounded_wait_selftest(int *status, long long limit_cycles, cudaStream_t s) {
    k_bounded_wait_selftest<<<1, 64, 0, s>>>(status, limit_cycles);
    return cudaGetLastError();
}

cudaError_t umma_init_weight_maps(WeightDev *w, const char **err) {
    w->tma_ok = false;
    if (w->qtype == kTypeF16) {
        // fp16 rows: 128-byte-swizzled boxes of 64 columns x 128 rows (forward) / 64 rows (backward), written straight
        // into the operand stages
        if (w->K % 128 != 0 || w->row_bytes == 0) return cudaSuccess;
        bool ok16 = encode_2d(&w->tm_q0_f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                              (uint64_t)w->row_bytes, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        ok16 = ok16 && encode_2d(&w->tm_q0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                                 (uint64_t)w->row_bytes, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B);
        if (!ok16) {
            if (err) *err = "cuTensorMapEncodeTiled failed for an fp16 weight tensor";
            return cudaErrorInvalidValue;
        }
        w->tm_hdr = w->tm_q1 = w->tm_q0;
        w->tm_hdr_f = w->tm_q1_f = w->tm_q0_f;
        w->tma_ok = true;
        return cudaSuccess;
    }
    if (w->qtype != kTypeQ4K && w->qtype != kTypeQ6K) return cudaSuccess;
    if (w->K % 256 != 0 || w->row_bytes == 0) return cudaSuccess;   // flat streams run on the CUDA-core path
    const int H = w->qtype == kTypeQ4K ? 16 : 32;
    bool ok = encode_2d(&w->tm_hdr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                        (uint64_t)w->row_bytes, H, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
    ok = ok && encode_2d(&w->tm_hdr_f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                         (uint64_t)w->row_bytes, H, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    ok = ok && encode_2d(&w->tm_q0_f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                         (uint64_t)w->row_bytes, 64, 128, CU_TENSOR_MAP_SWIZZLE_64B);
    if (w->qtype == kTypeQ6K)
        ok = ok && encode_2d(&w->tm_q1_f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                             (uint64_t)w->row_bytes, 32, 128, CU_TENSOR_MAP_SWIZZLE_32B);
    else
        w->tm_q1_f = w->tm_q0_f;
    ok = ok && encode_2d(&w->tm_q0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                         (uint64_t)w->row_bytes, 64, 64, CU_TENSOR_MAP_SWIZZLE_64B);
    if (w->qtype == kTypeQ6K)
        ok = ok && encode_2d(&w->tm_q1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                             (uint64_t)w->row_bytes, 32, 64, CU_TENSOR_MAP_SWIZZLE_32B);
    else
        w->tm_q1 = w->tm_q0;
    {   // whole super-blocks for the few-token tensor-core kernel
        const uint32_t bb = w->qtype == kTypeQ4K ? (uint32_t)kQ4KBlockBytes : (uint32_t)kQ6KDevBlockBytes;
        ok = ok && encode_2d(&w->tm_blk_f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                             (uint64_t)w->row_bytes, bb, 256, CU_TENSOR_MAP_SWIZZLE_NONE);
        ok = ok && encode_2d(&w->tm_blk_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->data, (uint64_t)w->row_bytes, (uint64_t)w->N,
                             (uint64_t)w->row_bytes, bb, 64, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (w->qtype == kTypeQ4K)      // whole packed rows for the few-token streaming kernel
        ok = ok && encode_2d(&w->tm_rows, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w->data, (uint64_t)w->row_bytes / 4, (uint64_t)w->N,
                             (uint64_t)w->row_bytes, 72, 16, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) {
        if (err) *err = "cuTensorMapEncodeTiled failed for a weight tensor";
        return cudaErrorInvalidValue;
    }
    w->tma_ok = true;
    return cudaSuccess;
}

static int eff_rows(const UmmaLaunch &L) { return L.rows > 0 ? L.rows : L.w->N; }

static int pick_splits(int tiles, int units, int T, int sm_count) {
    const int chunks = (T + kMaxTok - 1) / kMaxTok;
    int s = sm_count / (tiles * chunks > 0 ? tiles * chunks : 1);
    const int cap = units / 2 > 1 ? units / 2 : 1;
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    if (s > units) s = units;
    return s;
}

int umma_pick_splits(const WeightDev *w, int backward, int T, int sm_count) {
    const int tiles = backward ? w->K / kTileW : (w->N + kTileW - 1) / kTileW;
    const int units = backward ? (w->N + 63) / 64 : w->K / 128;
    return pick_splits(tiles, units, T, sm_count);
}

bool umma_group_ok(const UmmaLaunch *m, int n) {
    if (n < 1 || n > kMaxMembers) return false;
    for (int j = 0; j < n; j++) {
        const WeightDev *w = m[j].w;
        if (!w || !w->tma_ok || w->qtype != m[0].w->qtype || w->K != m[0].w->K) return false;
        if (m[j].rank > 64) return false;
        if (w->qtype == kTypeF16 && (!m[j].fp16 || m[j].rank > 0)) return false;      // fp16 rows: fp16 MMA operands, no adapter stage
        if (m[j].row_base < 0 || m[j].row_base + eff_rows(m[j]) > w->N) return false;
        if (m[j].backward != m[0].backward || m[j].fp16 != m[0].fp16 || m[j].T != m[0].T) return false;
        if (m[0].backward && m[j].out != m[0].out) return false;       // one shared dX
    }
    return true;
}

// CTA pairs pay off once the activation tile is the bulk of what an SM pulls from L2, and they halve the MMA
// instructions per weight; pair mode needs 16 token columns per CTA half (the knob is clamped to [32, 256])
static int pair_min_tokens() {
    static const int pair_min = [] {
        const int v = getenv("GT_PAIR_MIN") ? atoi(getenv("GT_PAIR_MIN")) : 256;
        return v < 32 ? 32 : (v > 256 ? 256 : v);
    }();
    return pair_min;
}

// every member qualifies for the few-token kernel (gt_umma_few.cu)
static bool few_group(const UmmaLaunch *m, int n) {
    for (int j = 0; j < n; j++)
        if (!umma_few_ok(m[j])) return false;
    return true;
}
bool umma_group_few(const UmmaLaunch *m, int n) { return few_group(m, n); }

int umma_group_splits(const UmmaLaunch *m, int n, int sm_count) {
    const bool bwd = m[0].backward != 0;
    if (few_group(m, n)) {
        // one launch per member, all with the same split count: forward sized for the members' tiles together (they run
        // back to back), backward for the longest contraction
        int tiles = 0, units = 0;
        for (int j = 0; j < n; j++) {
            int t, u;
            umma_few_shape(m[j], &t, &u);
            if (bwd) {
                tiles = t;
                units = u > units ? u : units;
            } else {
                tiles += t;
                units = u;
            }
        }
        // forward: a raw stage is eight weight stages, one per CTA is enough; backward: two (four weight stages)
        int sp = sm_count / (tiles > 0 ? tiles : 1);
        const int cap = bwd ? (units / 2 > 1 ? units / 2 : 1) : units;
        if (sp > cap) sp = cap;
        return sp < 1 ? 1 : sp;
    }
    const int tmax = m[0].T < kMaxTok ? m[0].T : kMaxTok;
    const bool pair = tmax >= pair_min_tokens();
    int tiles = 0, units = 0;
    for (int j = 0; j < n; j++) {
        const WeightDev *w = m[j].w;
        const int rows = eff_rows(m[j]);
        if (bwd) {
            units += (rows + 63) / 64;
            tiles = w->K / kTileW;
            if (pair) tiles = (tiles + 1) & ~1;
        } else {
            int t = (rows + kTileW - 1) / kTileW;
            if (pair) t = (t + 1) & ~1;
            tiles += t;
            units = w->K / 128;
        }
    }
    return pick_splits(tiles, units, m[0].T, sm_count);
}

// Members share T, math mode, direction, in_features and quantization type (umma_group_ok).  Forward: the activation
// operand and `splits` / `out_prefilled` come from member 0.  Backward: every member brings its own dY; `out` is shared.
// gate | up with the SwiGLU product in the epilogue: members 0 and 1 of the same shape and type, no split-K; either
// member's `out` may be null (nothing but the product is wanted), h16 receives SiLU(out0) * out1 as 16-bit values
bool umma_dual_ok(const UmmaLaunch *m, int sm_count) {
    if (!umma_group_ok(m, 2) || m[0].backward || few_group(m, 2)) return false;
    const WeightDev *a = m[0].w, *b = m[1].w;
    if (a->qtype == kTypeF16 || a->N != b->N || a->N % 64 != 0 || m[0].rows || m[1].rows) return false;
    if (m[0].rank > 32 || m[1].rank > 32 || m[0].out_prefilled || m[1].out_prefilled) return false;
    if (m[0].T <= 128) return false;      // the kernel's 256-row activation stages
    // one CTA per 64 features and token chunk, no split-K: worth it where those alone fill the GPU
    // (GT_FFN_DUAL_MIN_TILES, read at every call: a smaller bound, for tests on small tensors)
    const char *env = getenv("GT_FFN_DUAL_MIN_TILES");
    const int need = env ? atoi(env) : sm_count;
    return (a->N / 64) * ((m[0].T + kMaxTok - 1) / kMaxTok) >= need;
}

cudaError_t launch_umma_group(const UmmaLaunch *m, int n, cudaStream_t s, const char **err, const UmmaDual *dual) {
    if (dual && (n != 2 || !umma_dual_ok(m, 0))) {
        if (err) *err = "the two projections do not qualify for the dual forward";
        return cudaErrorInvalidValue;
    }
    if (!umma_group_ok(m, n)) {
        if (err) *err = "projections cannot share one launch (type, in_features, token count or TMA layout differ)";
        return cudaErrorInvalidValue;
    }
    const UmmaLaunch &L0 = m[0];
    if (L0.T <= 0) return cudaSuccess;
    const bool bwd = L0.backward != 0;
    if (!dual && few_group(m, n)) {
        // up to 128 tokens: the kernel with the weights on the wide operand, one launch per member; the adapter terms
        // follow on the exact rank-r kernels
        for (int j = 0; j < n; j++) {
            UmmaLaunch L = m[j];
            L.splits = L0.splits;
            if (bwd && j > 0) L.out_assign = 0;      // the members' products add up in one dX
            cudaError_t ce = launch_umma_few(L, s, err);
            if (ce != cudaSuccess) return ce;
        }
        for (int j = 0; j < n; j++) {
            const UmmaLaunch &L = m[j];
            if (L.rank <= 0 || !L.lora_act || !L.lora_w) continue;
            const int rows = eff_rows(L);
            if (L.ld_out != (bwd ? L.w->K : rows)) {      // the rank-r kernels take dense outputs
                if (err) *err = "few-token launch with an adapter needs a dense output tensor";
                return cudaErrorInvalidValue;
            }
            cudaError_t ce = bwd ? launch_lora_dx_fp32(L.lora_act, L.lora_w, L.out, L.lora_scale, L.T, L.w->K, L.rank, s)
                                 : launch_lora_delta_fp32(L.lora_act, L.lora_w, L.out, nullptr, L.T, rows, L.rank, L.lora_scale, L.lora_flag, s);
            if (ce != cudaSuccess) return ce;
        }
        return cudaSuccess;
    }
    Params p;
    memset(&p, 0, sizeof(p));
    const int tmax = L0.T < kMaxTok ? L0.T : kMaxTok;
    const bool pair = tmax >= pair_min_tokens();
    const int tb = pair ? (tmax + 31) & ~31 : (tmax + 15) & ~15;
    // pair mode: TMA box rows = half of an MMA's token columns (64 with four 128-column accumulators)
    static const int mtok = getenv("GT_MMA_TOK") ? atoi(getenv("GT_MMA_TOK")) : 256;
    p.t_box = pair ? (mtok == 128 ? 64 : 128) : (tb < 128 ? tb : 128);
    // one MMA per k-step (tokens <= its width): up to four partial accumulators side by side (see n_acc in the kernel)
    const int stride = (tb + 31) & ~31;
    const int mma_w = pair ? (mtok == 128 ? 128 : 256) : 512;
    // (up to 128 tokens on a single CTA: two sets of them, one per MMA issuer)
    const int need_cols = tb > mma_w ? tb
                                     : (!pair && stride <= 64 ? 8 * stride : (stride <= 128 ? 4 * stride : (stride <= 256 ? 2 * stride : stride)));
    int tc = 32;
    while (tc < need_cols) tc <<= 1;
    p.tmem_cols = tc;
    static const int par_ok = getenv("GT_MMA_PAR") ? atoi(getenv("GT_MMA_PAR")) : 1;
    p.par_ok = par_ok;
    const CUtensorMapDataType dt = L0.fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    p.n_members = n;
    int first = 0;
    for (int j = 0; j < n; j++) {
        const UmmaLaunch &L = m[j];
        const WeightDev *w = L.w;
        Member &M = p.m[j];
        // (64-row boxes: the backward's raw stages, and the dual forward's two half-tiles)
        M.tm_hdr = (L0.backward || dual) ? w->tm_hdr : w->tm_hdr_f;
        M.tm_q0 = (L0.backward || dual) ? w->tm_q0 : w->tm_q0_f;
        M.tm_q1 = (L0.backward || dual) ? w->tm_q1 : w->tm_q1_f;
        const int rows = eff_rows(L);
        M.row_base = L.row_base;
        if (bwd || j == 0) {
            const int cols = bwd ? rows : w->K;       // contraction length of the activation operand
            if (!encode_2d(&M.tm_act, dt, 2, L.act16, (uint64_t)cols, (uint64_t)L.T, (uint64_t)L.ld_act * 2, 64, (uint32_t)p.t_box,
                           CU_TENSOR_MAP_SWIZZLE_128B)) {
                if (err) *err = "cuTensorMapEncodeTiled failed for the activation operand";
                return cudaErrorInvalidValue;
            }
        } else {
            M.tm_act = p.m[0].tm_act;
        }
        M.out = L.out;
        M.ld_out = L.ld_out;
        M.bias = L.bias;
        M.N = rows;
        if (L.rank > 0 && L.lora_act && L.lora_w) {
            M.rank = L.rank;
            M.lora_w = L.lora_w;
            M.lora_act = L.lora_act;
            M.lora_scale = L.lora_scale;
            M.lora_flag = L.lora_flag;
        }
        int count;
        if (dual) {
            // every tile holds 64 rows of both members: all tiles are listed under member 0
            count = j == 0 ? rows / 64 : 0;
            if (pair && j == 0) count = (count + 1) & ~1;
            M.first = j == 0 ? 0 : 0x7fffffff;
            M.count = count;
            first += count;
            continue;
        }
        if (bwd) {
            count = (rows + 63) / 64;
        } else {
            count = (rows + kTileW - 1) / kTileW;
            if (pair) count = (count + 1) & ~1;      // a pair owns two adjacent tiles of ONE member; a padding tile is all out of range
        }
        M.first = first;
        M.count = count;
        first += count;
    }
    p.status = L0.status;
    p.trace = (long long *)L0.trace;
    p.T = L0.T;
    p.K = L0.w->K;
    p.units = bwd ? first : L0.w->K / 128;
    p.splits = L0.splits < 1 ? 1 : (L0.splits > p.units ? p.units : L0.splits);
    if (dual) {
        p.splits = 1;
        p.dual = 1;
        p.h16 = dual->h16;
        p.ld_h16 = dual->ld_h16;
    }
    // plain stores when one CTA owns each output tile and the output is to be written, not added to: a forward without
    // split-K, and a backward without split-K whose caller asked for "dX =" (out_assign)
    p.atomic_out = bwd ? ((p.splits > 1 || !L0.out_assign) ? 1 : 0) : (p.splits > 1 || L0.out_prefilled ? 1 : 0);
    // backward: one tile per 128 input columns; a CTA pair needs an even count (fp16 tensors may have in_features %
    // 256 == 128): the padding tile reads zero-filled weights and stores nothing
    int tiles = bwd ? L0.w->K / kTileW : first;
    if (bwd && pair) tiles = (tiles + 1) & ~1;
    dim3 grid(tiles, p.splits, (L0.T + kMaxTok - 1) / kMaxTok);
    const int qt = L0.w->qtype;
    if (qt == kTypeF16) return bwd ? launch_one<kTypeF16, __half, true>(p, grid, pair, s) : launch_one<kTypeF16, __half, false>(p, grid, pair, s);
    if (qt == kTypeQ4K) {
        if (!L0.fp16) return bwd ? launch_one<kTypeQ4K, __nv_bfloat16, true>(p, grid, pair, s) : launch_one<kTypeQ4K, __nv_bfloat16, false>(p, grid, pair, s);
        return bwd ? launch_one<kTypeQ4K, __half, true>(p, grid, pair, s) : launch_one<kTypeQ4K, __half, false>(p, grid, pair, s);
    }
    if (!L0.fp16) return bwd ? launch_one<kTypeQ6K, __nv_bfloat16, true>(p, grid, pair, s) : launch_one<kTypeQ6K, __nv_bfloat16, false>(p, grid, pair, s);
    return bwd ? launch_one<kTypeQ6K, __half, true>(p, grid, pair, s) : launch_one<kTypeQ6K, __half, false>(p, grid, pair, s);
}

cudaError_t launch_umma_gemm(const UmmaLaunch &L, cudaStream_t s, const char **err) {
    if (!L.w || !L.w->tma_ok) {
        if (err) *err = "weight tensor has no TMA maps (K % 256 != 0 or unsupported type)";
        return cudaErrorInvalidValue;
    }
    if (L.rank > 64) {
        if (err) *err = "fused LoRA update supports rank <= 64";
        return cudaErrorInvalidValue;
    }
    return launch_umma_group(&L, 1, s, err);
}

}  // namespace gt
