// Frozen-base Q4_K projection GEMMs for a few tokens (up to 64) on the sm_100a tensor cores.
//
//   forward   out[T, N]  (+)= act[T, K] * W[N, K]^T (+ bias)
//   backward  out[T, K]  (+)= act[T, N] * W[N, K]
//
// Replaces, for small batches, the same reference kernels as gt_umma_gemm.cu: gemm_q4_k_batch / gemm_q6_k_batch
// (launched at src/Glacier.Tune/Gpu/GpuLoraEngine.Forward.cs:83-129) and gemm_q4_k_bwd / gemm_q6_k_bwd
// (src/Glacier.Tune/Gpu/Kernels/tune_bwd.cu:193-332).
//
// Why a second kernel: a tcgen05.mma occupies the tensor pipe of its SM for about 128 clocks whatever the width N of
// its B operand (up to 256), because the A operand's 128 rows are what it walks.  gt_umma_gemm.cu puts the WEIGHTS on
// the A side (128 weight rows per MMA, tokens on the B side): right for 256-512 tokens, but with few tokens every
// 128 x 16 weights still cost 128 clocks, three times what streaming them from HBM takes.  Here the operands are
// swapped: the tokens (padded to 128 rows, the padding is zero-filled by TMA) are the A operand and 256 weight rows
// (forward) or 256 weight columns (backward) are the B operand, so an MMA covers twice the weights, and the weight
// stages are 32 deep (two MMAs each) so that four of them in flight fit beside a 112 KB ring of packed blocks:
//
//   D[128 tokens x 256] (TMEM, fp32)  +=  act[128 x 32] (SMEM via TMA)  x  Wtile[256 x 32] (SMEM, dequantized 16-bit)
//
// The second bound at few tokens is the rate at which the TMA unit takes row requests (about one per three clocks,
// whatever the row's size): the packed weights therefore arrive as WHOLE super-blocks (one 144- or 224-byte request
// per row and 256 weights, where gt_umma_gemm.cu fetches header and quants of half a block separately), and the
// activations as 128-byte rows (one tile of 64 contraction elements feeds two weight stages).
//
// Warp roles (640 threads):
//   warp 0        TMA producer of the packed weight blocks (one tiled copy per raw stage)
//   warp 19       TMA producer of the 16-bit activation tiles
//   warps 1, 18   tcgen05.mma issuers; issuer i takes the operand stages n = i (mod 2) and owns accumulator i (TMEM
//                 columns 256 i ..), so the two never wait for each other and every accumulator receives its MMAs from
//                 one thread in a fixed order (results do not change from run to run); warp 1 owns the TMEM allocation
//   warps 2-17    two groups of 8 warps; a group dequantizes PAIRS of weight stages (two 32-weight sub-blocks of the same
//                 rows: one thread, one row, one header decode, 64 weights), the groups take alternate pairs;
//                 afterwards all 16 run the epilogue (tcgen05.ld of both accumulators -> sum -> bias -> store / atomic)
//
// forward : raw stage = 256 rows x one super-block (256 weights) = eight weight stages, one per 32-weight sub-block;
//           group g takes the sub-block pairs g and g + 2, so both groups read every raw stage.  The weight tile is K-major
//           with 64-byte rows (64-byte swizzle); the activation tile K-major with 128-byte rows (128-byte swizzle).
// backward: raw stage = 64 rows x one super-block (256 columns) = two weight stages of 32 rows = one pair (the groups
//           take alternate raw stages); the weight tile is
//           the MN-major B operand (four images of 32 rows x 64 columns, 128-byte swizzle), the dY tile as in the
//           forward.  No transposed copy of W is formed.
//
// Split-K over blockIdx.y fills the GPU (a 18944 x 3584 tensor is 74 row tiles); partial tiles are added with fp32
// atomics into an output the caller has pre-filled (bias or zero), exactly like the split-K mode of gt_umma_gemm.cu.
// The adapter term is not fused here: the caller adds it with the exact rank-r kernels.
// Every mbarrier wait is bounded; on a timeout the CTA records a code in status[0], all roles leave their loops,
// TMEM is released and the kernel returns.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "gt_internal.h"
#include "gt_ptx.cuh"
#include "gt_quant.cuh"

namespace gt {

namespace {

constexpr int kTok = 128;            // token rows of the A operand (UMMA M)
constexpr int kTileN = 256;          // weight rows (forward) / columns (backward) per CTA (UMMA N)
constexpr int kDepth = 32;           // contraction elements per weight stage
constexpr int kMaxSlots = 8;         // weight stages in flight: 8 where they fit beside two raw stages, else 4
constexpr int kMaxXSlots = 6;        // activation tiles in flight (64 contraction elements = two weight stages each): 24 KB of
                                     // 32- or 64-row tiles, 48 KB of 128-row tiles; their L2 latency is several stage times
constexpr int kWSlotBytes = kTileN * kDepth * 2;      // 16 KiB
constexpr int kOffBarF = 224 * 1024;
constexpr int kMaxRawF = 12;
constexpr int kBarBytesF = 512;
constexpr int kSmemF = kOffBarF + kBarBytesF + 1024;
constexpr int kThreadsF = 640;
constexpr int kIssuer2 = 18, kActWarp = 19;

constexpr int kBRawFull = 0, kBRawEmpty = kMaxRawF, kBFull = 2 * kMaxRawF, kBEmpty = kBFull + kMaxSlots, kBXFull = kBEmpty + kMaxSlots,
              kBXEmpty = kBXFull + kMaxXSlots, kBAcc = kBXEmpty + kMaxXSlots, kNumBarsF = kBAcc + 1;
constexpr int kOffTmemF = kNumBarsF * 8, kOffAbortF = kOffTmemF + 4;
static_assert(kOffAbortF + 4 <= kBarBytesF, "barrier region too small");

struct FewParams {
    CUtensorMap tm_blk;                 // packed weight bytes, boxes of one super-block x 256 rows (forward) / 64 rows (backward)
    CUtensorMap tm_act;                 // 16-bit activations, boxes of 64 elements x 128 token rows, 128-byte swizzle
    float *out;
    const float *bias;
    int *status;
    long long *trace;                   // optional timeline of CTA (0,0): [12 rows][128] SM clock values, or null
    int T, K, N;                        // N = rows of the window
    int row_base, ld_out;
    int units, splits;                  // raw stages along the contraction, K splits
    int atomic_out;
};

enum { kFewProducer = 600, kFewMma = 700, kFewDequant = 800, kFewEpilogue = 900 };

// Shared memory: [activation tiles | weight stages | ring of packed blocks | barriers].  XROWS = token rows an
// activation tile holds (32, 64 or 128; the MMA always reads 128 rows: with fewer, the rest of its A operand is whatever
// follows the tile in shared memory, and only ever reaches accumulator rows that are not stored).  With eight weight
// slots a dequant group owns two pairs of them: it fills one pair while the MMAs of the other are still queued.
template <int QT, typename T16, bool BWD, int XROWS>
__global__ void __launch_bounds__(kThreadsF, 1) k_umma_few(const __grid_constant__ FewParams p) {
    using QS = QuantStage<QT>;
    constexpr int BB = QS::kBlockBytes;             // bytes of a super-block = row pitch of a raw stage
    constexpr int kRows = BWD ? 64 : kTileN;        // weight rows of a raw stage
    constexpr int kRawStageBytes = (kRows * BB + 1023) & ~1023;
    constexpr int kPerRaw = BWD ? 2 : 8;            // weight stages per raw stage
    constexpr int kXSlotBytes = XROWS * 128;
    constexpr int kXSlots = XROWS == 32 ? 6 : 3;
    constexpr int kOffXf = 0;
    constexpr int kOffWf = kOffXf + kXSlots * kXSlotBytes;
    constexpr int kSlots = kOffWf + kMaxSlots * kWSlotBytes + 2 * kRawStageBytes <= kOffBarF ? kMaxSlots : 4;
    constexpr int kOffRawF = kOffWf + kSlots * kWSlotBytes;
    constexpr int kRawBudgetF = kOffBarF - kOffRawF;
    static_assert(kOffWf + 128 * 128 <= kOffRawF, "the MMA's 128-row view of the last activation tile stays inside the buffer");
    constexpr int kFit = kRawBudgetF / kRawStageBytes < kMaxRawF ? kRawBudgetF / kRawStageBytes : kMaxRawF;
    // backward: a dequant group visits every second raw stage; an even ring keeps each slot with the same two groups, who
    // then see every phase of its barriers (a parity wait must not skip a phase)
    constexpr int kNumRaw = BWD ? (kFit & ~1) : kFit;
    static_assert(kNumRaw >= 2, "raw ring too small");
    constexpr uint32_t kFmt = std::is_same<T16, __half>::value ? 0u : 1u;

    extern __shared__ uint8_t smem_dyn[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBarF;
    auto bar = [&](int slot) -> uint32_t { return bar0 + 8u * (uint32_t)slot; };
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + kOffBarF + kOffAbortF);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kOffBarF + kOffTmemF);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int u0 = (int)((int64_t)p.units * split / p.splits);
    const int u1 = (int)((int64_t)p.units * (split + 1) / p.splits);
    const int nu = u1 - u0;
    const int n_total = nu * kPerRaw;       // weight stages of this CTA (>= 2: either issuer has work)
    const int n_x = n_total / 2;            // activation tiles

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumRaw; i++) {
            mbar_init(bar(kBRawFull + i), 1);
            mbar_init(bar(kBRawEmpty + i), BWD ? 8 : 16);      // one arrival per warp that read the stage (backward: one group)
        }
        for (int i = 0; i < kSlots; i++) {
            mbar_init(bar(kBFull + i), 8);                     // the eight warps of the slot's group
            mbar_init(bar(kBEmpty + i), 1);                    // tcgen05.commit of the stage's MMAs
        }
        for (int i = 0; i < kXSlots; i++) {
            mbar_init(bar(kBXFull + i), 1);                    // the producer's arrival with the tile's bytes
            mbar_init(bar(kBXEmpty + i), 2);                   // tcgen05.commit of either issuer (one weight stage each)
        }
        mbar_init(bar(kBAcc), 2);                              // both issuers commit to it
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_act);
        tma_prefetch_desc(&p.tm_blk);
    }
    if (warp == 1) {
        tmem_alloc(sbase + kOffBarF + kOffTmemF, 512u);
        tmem_relinquish();
    }
    pdl_wait();
    pdl_trigger();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    auto trace = [&](int row, int idx) {
        if (tracing && idx < 128) p.trace[row * 128 + idx] = clock64();
    };
    if (threadIdx.x == 0) trace(11, 0);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer of the packed weights
        if (lane == 0) {
            bool ok = true;
            for (int u = u0; u < u1 && ok; u++) {
                const int r = u - u0, ri = r % kNumRaw;
                if (r >= kNumRaw)
                    ok = mbar_wait_bounded(bar(kBRawEmpty + ri), (uint32_t)((r - kNumRaw) / kNumRaw) & 1u, abort_flag, p.status, kFewProducer + 1);
                if (!ok) break;
                const uint32_t rbar = bar(kBRawFull + ri);
                // forward: super-block u of rows tile * 256 ..; backward: super-block `tile` of rows 64 u ..
                const int xb = (BWD ? tile : u) * BB;
                const int row0 = p.row_base + (BWD ? u * 64 : tile * kTileN);
                mbar_arrive_expect_tx(rbar, (uint32_t)(kRows * BB));
                tma_load_2d(sbase + kOffRawF + ri * kRawStageBytes, &p.tm_blk, xb, row0, rbar);
                trace(0, r);
            }
        }
    } else if (warp == kActWarp) {
        // ------------------------------------------------------------------ TMA producer of the activation tiles
        if (lane == 0) {
            bool ok = true;
            for (int m = 0; m < n_x && ok; m++) {
                const int xi = m % kXSlots;
                if (m >= kXSlots)
                    ok = mbar_wait_bounded(bar(kBXEmpty + xi), (uint32_t)((m - kXSlots) / kXSlots) & 1u, abort_flag, p.status, kFewProducer + 2);
                if (!ok) break;
                // tile m = contraction elements 64 m .. of this CTA's range (forward: 256 per raw stage, backward: 64)
                const int c0 = (BWD ? u0 * 64 : u0 * 256) + m * 64;
                mbar_arrive_expect_tx(bar(kBXFull + xi), (uint32_t)kXSlotBytes);
                tma_load_2d(sbase + kOffXf + xi * kXSlotBytes, &p.tm_act, c0, 0, bar(kBXFull + xi));
                trace(1, m);
            }
        }
    } else if (warp == 1 || warp == kIssuer2) {
        // ------------------------------------------------------------------ two independent MMA issuers
        if (lane == 0) {
            const int who = warp == 1 ? 0 : 1;
            bool ok = true;
            // descriptors as (lo, hi) words: lo = (addr >> 4) | (LBO >> 4) << 16, hi = (SBO >> 4) | version 1 << 14 | layout << 29
            constexpr uint32_t kHi64 = (512u >> 4) | (1u << 14) | (4u << 29);        // K-major, 64-byte swizzle
            constexpr uint32_t kHi128 = (1024u >> 4) | (1u << 14) | (2u << 29);      // MN-major, 128-byte swizzle
            constexpr uint32_t kBHi = BWD ? kHi128 : kHi64;
            constexpr uint32_t kBLoField = (BWD ? (4096u >> 4) : 1u) << 16;          // MN-major: LBO = stride between 64-column images
            constexpr uint32_t kBStep = (BWD ? 2048u : 32u) >> 4;                    // per k-step advance of the B operand
            const uint32_t idesc = umma_idesc_f16(kFmt, 0u, BWD ? 1u : 0u, (uint32_t)kTileN, (uint32_t)kTok);
            const uint32_t d_tmem = tmem_base + (uint32_t)(who * kTileN);
            for (int n = who; n < n_total && ok; n += 2) {
                const int si = n % kSlots, m = n >> 1, xi = m % kXSlots;
                ok = mbar_wait_bounded(bar(kBXFull + xi), (uint32_t)(m / kXSlots) & 1u, abort_flag, p.status, kFewMma + 2);
                if (!ok) break;
                ok = mbar_wait_bounded(bar(kBFull + si), (uint32_t)(n / kSlots) & 1u, abort_flag, p.status, kFewMma + 1);
                if (!ok) break;
                tc_fence_after_sync();
                if (who == 0) trace(8, n >> 1);
                // this issuer's half of the activation tile: k-steps 2 who, 2 who + 1 of its 128-byte rows
                const uint32_t a_lo = (((sbase + kOffXf + xi * kXSlotBytes) & 0x3FFFFu) >> 4) + (uint32_t)(who * 4) | (1u << 16);
                const uint32_t b_lo = (((sbase + kOffWf + si * kWSlotBytes) & 0x3FFFFu) >> 4) | kBLoField;
                umma_f16_ss_lohi<false>(d_tmem, a_lo, kHi128, b_lo, kBHi, idesc, n == who ? 0u : 1u);
                umma_f16_ss_lohi<false>(d_tmem, a_lo + 2, kHi128, b_lo + kBStep, kBHi, idesc, 1u);
                umma_commit(bar(kBEmpty + si));
                umma_commit(bar(kBXEmpty + xi));
                if (who == 0) trace(9, n >> 1);
            }
            if (ok) umma_commit(bar(kBAcc));
        }
    } else {
        // ------------------------------------------------------------------ dequant warps, then epilogue
        const int dt = (threadIdx.x - 64) & 255;        // thread index inside its 8-warp group
        const int g2 = (warp - 2) >> 3;                 // group 0 / 1
        const int g4 = (warp - 2) >> 2;                 // column group of the epilogue
        bool ok = true;
        // weight stage n lives in slot n % kSlots; pair P = stages 2 P, 2 P + 1 belongs to group P % 2
        auto wait_slot = [&](int n) -> bool {
            if (n < kSlots) return true;
            return mbar_wait_bounded(bar(kBEmpty + n % kSlots), (uint32_t)((n - kSlots) / kSlots) & 1u, abort_flag, p.status, kFewDequant + 2);
        };
        auto publish_pair = [&](int n) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar(kBFull + n % kSlots));
                mbar_arrive(bar(kBFull + (n + 1) % kSlots));
            }
        };
        auto w_slot = [&](int n) -> uint32_t { return sbase + kOffWf + (uint32_t)((n % kSlots) * kWSlotBytes); };
        if (!BWD) {
            // pair q (0..3) of raw stage ui = sub-blocks 2 q, 2 q + 1 of the super-block (32-weight groups 2 (q & 1) and
            // 2 (q & 1) + 1 of half q >> 1), all 256 rows; a thread owns row dt.  Tile image: row = weight row, 64 bytes =
            // 32 consecutive k, 16-byte chunks XOR (row >> 1) & 3.
            const int row = dt;
            for (int ui = 0; ui < nu && ok; ui++) {
                const int ri = ui % kNumRaw;
                ok = mbar_wait_bounded(bar(kBRawFull + ri), (uint32_t)(ui / kNumRaw) & 1u, abort_flag, p.status, kFewDequant + 1);
                if (!ok) break;
                const uint8_t *rr = smem + kOffRawF + ri * kRawStageBytes + row * BB;
                if (dt == 0 && g2 == 0) trace(2, ui);
                for (int pp = 0; pp < 2 && ok; pp++) {
                    const int q = 2 * pp + g2, half = q >> 1, n = 8 * ui + 2 * q;
                    ok = wait_slot(n) && wait_slot(n + 1);
                    if (!ok) break;
                    if (dt == 0 && g2 == 0) trace(3, 2 * ui + pp);
#pragma unroll
                    for (int e = 0; e < 2; e++)
                        dequant32_to_swizzled_row<QT, T16>(rr + QS::hdr_x(half), rr + QS::q0_x(half), rr + QS::q1_x(half), 0, 0, half,
                                                           2 * (q & 1) + e, w_slot(n + e) + (uint32_t)(row * 64), (row >> 1) & 3, 0);
                    publish_pair(n);
                    if (dt == 0 && g2 == 0) trace(4, 2 * ui + pp);
                }
                if (!ok) break;
                if (lane == 0) mbar_arrive(bar(kBRawEmpty + ri));
            }
        } else {
            // raw stage ui = 64 rows x 256 columns = the pair of weight stages 2 ui (rows 0-31), 2 ui + 1 (rows 32-63); the
            // groups take alternate raw stages.  Tile image j (64 columns): row = weight row, 128 bytes = 64 consecutive k,
            // chunks XOR (row & 7).  A thread owns one row of one image: the two 32-weight groups of its 64 columns.
            const int row = dt & 63, j = dt >> 6, r = row & 31, st = row >> 5, hb = j >> 1;
            for (int ui = g2; ui < nu && ok; ui += 2) {
                const int ri = ui % kNumRaw;
                ok = mbar_wait_bounded(bar(kBRawFull + ri), (uint32_t)(ui / kNumRaw) & 1u, abort_flag, p.status, kFewDequant + 1);
                if (!ok) break;
                if (dt == 0 && g2 == 0) trace(2, ui >> 1);
                const int n = 2 * ui;
                ok = wait_slot(n) && wait_slot(n + 1);
                if (!ok) break;
                if (dt == 0 && g2 == 0) trace(3, ui >> 1);
                const uint8_t *rr = smem + kOffRawF + ri * kRawStageBytes + row * BB;
                const uint32_t w_addr = w_slot(n + st) + (uint32_t)(j * 4096 + r * 128);
#pragma unroll
                for (int e = 0; e < 2; e++)
                    dequant32_to_swizzled_row<QT, T16>(rr + QS::hdr_x(hb), rr + QS::q0_x(hb), rr + QS::q1_x(hb), 0, 0, hb, 2 * (j & 1) + e,
                                                       w_addr, r & 7, 4 * e);
                publish_pair(n);
                if (dt == 0 && g2 == 0) trace(4, ui >> 1);
                if (lane == 0) mbar_arrive(bar(kBRawEmpty + ri));
            }
        }
        // epilogue: TMEM lane = token, TMEM column = weight row (forward) / column (backward) of this tile
        if (ok) ok = mbar_wait_bounded(bar(kBAcc), 0u, abort_flag, p.status, kFewEpilogue + 1, 16000000000ll);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-collective: take the epilogue only as a whole warp
        if (threadIdx.x == 64) trace(11, 1);
        const int quad = warp & 3;
        if (ok && quad * 32 < p.T) {
            tc_fence_after_sync();
            const int t = quad * 32 + lane;
            const int olim = BWD ? p.K : p.N;
            const bool vec = (p.ld_out & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
#pragma unroll 1
            for (int c = 2 * g4; c < 2 * g4 + 2; c++) {
                uint32_t v[32], w2[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(kTileN + c * 32), w2);
                tmem_ld_wait();
                const int o0 = tile * kTileN + c * 32;
                if (t < p.T && o0 < olim) {
                    float *dst = p.out + (int64_t)t * p.ld_out + o0;
                    if (p.atomic_out && vec && o0 + 32 <= olim) {
                        // four partial sums per reduction (16-byte aligned: ld_out % 4 == 0, o0 % 32 == 0)
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i),
                                         "f"(__uint_as_float(v[i]) + __uint_as_float(w2[i])),
                                         "f"(__uint_as_float(v[i + 1]) + __uint_as_float(w2[i + 1])),
                                         "f"(__uint_as_float(v[i + 2]) + __uint_as_float(w2[i + 2])),
                                         "f"(__uint_as_float(v[i + 3]) + __uint_as_float(w2[i + 3]))
                                         : "memory");
                    } else if (p.atomic_out) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (o0 + i < olim) atomicAdd(dst + i, __uint_as_float(v[i]) + __uint_as_float(w2[i]));
                    } else if (vec && o0 + 32 <= olim) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 o;
                            o.x = __uint_as_float(v[i]) + __uint_as_float(w2[i]);
                            o.y = __uint_as_float(v[i + 1]) + __uint_as_float(w2[i + 1]);
                            o.z = __uint_as_float(v[i + 2]) + __uint_as_float(w2[i + 2]);
                            o.w = __uint_as_float(v[i + 3]) + __uint_as_float(w2[i + 3]);
                            if (!BWD && p.bias) {
                                const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + o0 + i));
                                o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                            }
                            *reinterpret_cast<float4 *>(dst + i) = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (o0 + i < olim)
                                dst[i] = __uint_as_float(v[i]) + __uint_as_float(w2[i]) + ((!BWD && p.bias) ? p.bias[o0 + i] : 0.f);
                    }
                }
            }
        }
    }

    if (threadIdx.x == 64) trace(11, 2);
    if (*abort_flag) {
        // give loads that were already issued time to land before the CTA's shared memory is released
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, 512u);
    }
}

template <int QT, typename T16, bool BWD, int XROWS>
cudaError_t launch_few_x(const FewParams &p, dim3 grid, cudaStream_t s) {
    static PerDeviceOnce configured;
    auto kern = k_umma_few<QT, T16, BWD, XROWS>;
    cudaError_t ce = per_device_once(configured, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF); });
    if (ce != cudaSuccess) return ce;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreadsF);
    cfg.dynamicSmemBytes = kSmemF;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}
template <int QT, typename T16, bool BWD>
cudaError_t launch_few_variant(const FewParams &p, dim3 grid, cudaStream_t s) {
    if (p.T <= 32) return launch_few_x<QT, T16, BWD, 32>(p, grid, s);
    return p.T <= 64 ? launch_few_x<QT, T16, BWD, 64>(p, grid, s) : launch_few_x<QT, T16, BWD, 128>(p, grid, s);
}

}  // namespace

int umma_few_max_tokens() {
    static const int v = [] {
        const char *e = getenv("GT_FEW_MAX_T");
        const int n = e ? atoi(e) : 64;      // beyond 64 tokens the kernel in gt_umma_gemm.cu is as fast
        return n < 0 ? 0 : (n > kTok ? kTok : n);
    }();
    return v;
}

bool umma_few_ok(const UmmaLaunch &L) {
    const WeightDev *w = L.w;
    // Q4_K only: a Q6_K stage ring (224-byte blocks) leaves room for four weight stages and two raw stages, and measured
    // slower than gt_umma_gemm.cu's 128-token variant (down projection forward at 16 tokens: 43 us against 34 us per call;
    // dX 30 us either way)
    if (!w || !w->tma_ok || w->qtype != kTypeQ4K) return false;
    if (L.T < 1 || L.T > umma_few_max_tokens() || (w->K % 256) != 0) return false;
    const int rows = L.rows > 0 ? L.rows : w->N;
    // the contraction must give either MMA issuer a stage: forward K >= 128 always does; backward needs 64 rows
    return rows >= 1 && (L.ld_act % 8) == 0 && (reinterpret_cast<uintptr_t>(L.act16) & 15) == 0;
}

// tiles / contraction units of one member (the caller sums tiles over the members that share a launch's split count)
void umma_few_shape(const UmmaLaunch &L, int *tiles, int *units) {
    const int rows = L.rows > 0 ? L.rows : L.w->N;
    if (L.backward) {
        *tiles = L.w->K / kTileN;
        *units = (rows + 63) / 64;
    } else {
        *tiles = (rows + kTileN - 1) / kTileN;
        *units = L.w->K / 256;
    }
}

// One member.  `splits` > 1 or out_prefilled (forward) / !out_assign (backward): partial tiles are added atomically into
// an output the caller prepared; otherwise every tile is stored once (forward: + bias).
cudaError_t launch_umma_few(const UmmaLaunch &L, cudaStream_t s, const char **err) {
    if (!umma_few_ok(L)) {
        if (err) *err = "projection does not qualify for the few-token kernel";
        return cudaErrorInvalidValue;
    }
    const WeightDev *w = L.w;
    const bool bwd = L.backward != 0;
    FewParams p;
    memset(&p, 0, sizeof(p));
    p.tm_blk = bwd ? w->tm_blk_b : w->tm_blk_f;
    const int rows = L.rows > 0 ? L.rows : w->N;
    const int cols = bwd ? rows : w->K;       // contraction length of the activation operand
    if (!tmap_encode_2d(&p.tm_act, L.fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, L.act16, (uint64_t)cols,
                        (uint64_t)L.T, (uint64_t)L.ld_act * 2, 64, L.T <= 32 ? 32 : (L.T <= 64 ? 64 : kTok), CU_TENSOR_MAP_SWIZZLE_128B)) {
        if (err) *err = "cuTensorMapEncodeTiled failed for the activation operand";
        return cudaErrorInvalidValue;
    }
    p.out = L.out;
    p.bias = L.bias;
    p.status = L.status;
    p.trace = (long long *)L.trace;
    p.T = L.T;
    p.K = w->K;
    p.N = rows;
    p.row_base = L.row_base;
    p.ld_out = L.ld_out;
    int tiles, units;
    umma_few_shape(L, &tiles, &units);
    p.units = units;
    p.splits = L.splits < 1 ? 1 : (L.splits > units ? units : L.splits);
    p.atomic_out = bwd ? ((p.splits > 1 || !L.out_assign) ? 1 : 0) : ((p.splits > 1 || L.out_prefilled) ? 1 : 0);
    const dim3 grid(tiles, p.splits);
    if (!L.fp16) return bwd ? launch_few_variant<kTypeQ4K, __nv_bfloat16, true>(p, grid, s) : launch_few_variant<kTypeQ4K, __nv_bfloat16, false>(p, grid, s);
    return bwd ? launch_few_variant<kTypeQ4K, __half, true>(p, grid, s) : launch_few_variant<kTypeQ4K, __half, false>(p, grid, s);
}

}  // namespace gt
