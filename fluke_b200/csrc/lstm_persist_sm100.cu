// lstm_persist_sm100.cu -- one persistent launch per factored-LSTM layer.
//
// The per-timestep launches of lstm_sm100.cu re-load the gate weights from L2 and pay two
// launch latencies every step. Here the whole recurrence of a layer runs in ONE cooperative
// launch whose CTAs stay resident for all T timesteps:
//
//   gate CTAs   (PAIR of 128-chunk row tiles) x (slice of UNITS hidden units). The slice's four
//               gate weight blocks [4*UNITS, 2R] f16 stay in shared memory; the cell state of
//               the slice stays in REGISTERS for the whole layer. The two row tiles of the pair
//               are independent recurrences that the CTA works on alternately, each with its own
//               accumulator in tensor memory, its own operand buffers and its own four epilogue
//               warps: while one tile's hidden state travels to the worker and back, the other
//               tile computes. Per tile and step: the x_down half of the contraction is issued
//               as soon as its tile is there, the hh_down half when the projected hidden state
//               arrives; gates, cell update and the int8 hidden slice follow, written to h_out[t]
//               and published with a counter.
//   worker CTAs (row tile) x (half of the tile's ROWS). The int8 down-projection weights (all
//               R rows) stay in shared memory. Per step: wait until all slices of the tile have
//               published h_{t-1}, TMA-load the worker's 64 rows of it, tcgen05 kind::i8
//               contraction, scale, round to f16 (as the two-kernel form does) and publish its
//               rows of hh_down[tile]. The split is over rows, not projection columns, because
//               the load of h is what the step waits for longest: a worker takes in 64 x H bytes
//               instead of 128 x H. The MMA still has M = 128; the upper 64 rows of its A operand
//               are whatever lies behind the valid rows in shared memory, and the accumulator
//               rows they produce are never read.
//
// Exchange between CTAs goes through L2 (h_out itself and a [B,R] f16 buffer) with per-tile
// counters: writers store, meet at a CTA-scope barrier, then one thread fences at GPU scope and
// increments the counter; readers poll with ld.acquire, then fence.proxy.async before the TMA
// load of the freshly written data. The launch is cooperative only to guarantee that all CTAs
// are co-resident (no grid.sync). Every wait is bounded; a timeout raises a global abort word
// that all CTAs observe.
//
// Arithmetic is that of lstm_step_kernel and of the dequant GEMM epilogue, except that the two
// K halves are accumulated x_down first and tanh is evaluated with the fast exponential (see
// lstm_cell_pair).
#include <fluke/fluke.h>

#include "fluke_sm100.h"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <cuda_fp16.h>

namespace fluke_sm100 {
namespace {

constexpr int kPThreads = 320;          // warp 0 producer, warp 1 MMA, warps 2-5 / 6-9 epilogue
constexpr int kPRank = 128;             // factor rank the kernel is built for
constexpr int kPMaxHKB = 8;             // hidden K blocks of 128 bytes: H <= 1024
constexpr long long kPStaggerCycles = 9000;  // head start of a pair's first row tile over its second: about
                                        // half a step (a step is 14-19 thousand cycles); measured flat from 7 to 12 thousand

struct PersistDev {
    int T, B, H;               // B: chunks handled by this launch
    int b_stride;              // chunks per timestep plane of h_out (the full batch)
    int reverse;
    int n_tiles, n_pairs, n_slices;
    int nkb_h;                 // H / 128
    const float *bias;         // [4H]
    const float *dn_scale;     // [R]
    float *c;                  // [B,H]
    int8_t *h_out;             // [T,B,H]
    __half *hh_down;           // [B,R]
    unsigned int *flags;       // [0,n_tiles): h_ready, [n_tiles,2n_tiles): hh_ready, [2n_tiles]: abort
    long long *trace;          // trace builds only: [T][8] SM-clock stamps of CTA 0 and of the first worker
};

// Builds with -DFLUKE_SM100_TRACE (never the library's default build) record time stamps at the
// hand-over points of every step into a buffer set with fluke_sm100_lstm_set_trace.
#ifdef FLUKE_SM100_TRACE
static long long *g_persist_trace = nullptr;
inline long long *trace_buffer() { return g_persist_trace; }
#else
inline long long *trace_buffer() { return nullptr; }
#endif

// UNITS: hidden units per gate CTA. WPT: worker CTAs per row tile, 2 (each takes 64 of the
// tile's rows) or 1 (the whole tile; for the wide configuration, where the SMs go to twice as
// many row tiles instead).
template <int UNITS, int WPT>
struct PersistSmem {
    static_assert(WPT == 1 || WPT == 2, "one or two workers per row tile");
    // tensor memory: one accumulator of 4*UNITS columns per tile of the pair (gate role); the
    // worker's accumulator has kPRank columns
    static constexpr int kAccStride = (4 * UNITS <= 128) ? 128 : 256;
    static constexpr int kTmemCols = 2 * kAccStride;
    // gate role
    static constexpr int kWKB = 4 * UNITS * 128;           // one K block of the four gate slices
    static constexpr int kOffW = 0;                         // 4 K blocks
    static constexpr int kOffAhh = 4 * kWKB;                // per tile: 2 K blocks x 16 KB
    static constexpr int kOffX = kOffAhh + 2 * 32768;       // per tile: 2 K blocks x 16 KB
    static constexpr int kOffBias = kOffX + 2 * 32768;      // 4 x UNITS floats
    static constexpr int kGateBytes = kOffBias + 4 * UNITS * 4;
    // worker role
    static constexpr int kWorkerRows = 128 / WPT;           // rows of the tile a worker projects
    static constexpr int kMaxHKB = (WPT == 2) ? kPMaxHKB : 6;  // hidden K blocks the layout holds
    static constexpr int kDnKB = kPRank * 128;              // R projection rows x 128 B
    static constexpr int kOffDn = 0;
    static constexpr int kOffH = kPMaxHKB * kDnKB;
    static constexpr int kHKB = kWorkerRows * 128;          // the worker's rows of h x 128 B per K block
    static constexpr int kStageBytes = 2 * kWorkerRows * 128;  // outgoing hh_down rows: 2 column halves
    // WPT == 2: the MMA reads 128 rows per K block, 64 of them behind the worker's own: one block
    // of slack after the last, then the staging tile. WPT == 1: the staging tile sits in the part
    // of the weight area that at most 6 K blocks leave free.
    static constexpr int kOffStage = (WPT == 2) ? kOffH + (kPMaxHKB + 1) * kHKB : kMaxHKB * kDnKB;
    static constexpr int kWorkerBytes = (WPT == 2) ? kOffStage + kStageBytes : kOffH + kMaxHKB * kHKB;
    static_assert(WPT == 2 || kOffStage + kStageBytes <= kOffH, "staging tile overlaps the h tile");
    static constexpr int kData = ((kGateBytes > kWorkerBytes ? kGateBytes : kWorkerBytes) + 15) / 16 * 16;
    static constexpr int kOffBars = kData;
    static constexpr int kNumBars = 12;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;
    static constexpr int kDynamic = kOffMisc + 16 + 1024;
    static_assert(kDynamic <= 232448, "shared memory budget of one CTA exceeded");
};

// Barrier over a set of warps built on an mbarrier so that, unlike bar.sync, the wait is
// bounded: one arrival per warp (release at CTA scope), then every thread waits for the phase.
__device__ __forceinline__ bool warps_barrier(uint64_t *bar, uint32_t parity, int lane,
                                              volatile int *abort_flag) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    return mbar_wait(bar, parity, abort_flag, 60);
}

// Publishes everything the CTA's epilogue warps stored before their barrier: GPU-scope fence by
// one thread (cumulative over the writes it observed through the barrier), then the increment.
__device__ __forceinline__ void publish(unsigned int *counter) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// The cell update of two adjacent hidden units of one row, in packed f32x2 arithmetic where the
// instruction set has it. gi..go: the accumulator bits (f32) of the four gates of units u, u+1;
// bi..bo: their biases; c: the two cell values, updated in place. Returns the two int8 codes of
// h in bits 0-7 and 8-15.
//   gates   i, f, o = clamp(0.2 (acc + b) + 0.5, 0, 1) as one saturating fma each,
//           g = clamp(acc + b, -1, 1)
//   cell    c = fma(f, c, i * g)
//   hidden  h = o * tanh(c), tanh as 1 - 2 / (exp(2c) + 1) with the fast exponential (absolute
//           error ~1e-7, far below one int8 code); code = trunc(127 h +- 0.5)
__device__ __forceinline__ float p_sat_fma(float x, float a, float b) {
    float y;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(x), "f"(a), "f"(b));
    return y;
}
__device__ __forceinline__ uint32_t lstm_cell_pair(uint32_t gi0, uint32_t gi1, uint32_t gf0, uint32_t gf1,
                                                   uint32_t gg0, uint32_t gg1, uint32_t go0, uint32_t go1,
                                                   float2 bi, float2 bf, float2 bg, float2 bo, float2 &c) {
    const float2 pi = add2(make_float2(__uint_as_float(gi0), __uint_as_float(gi1)), bi);
    const float2 pf = add2(make_float2(__uint_as_float(gf0), __uint_as_float(gf1)), bf);
    const float2 pg = add2(make_float2(__uint_as_float(gg0), __uint_as_float(gg1)), bg);
    const float2 po = add2(make_float2(__uint_as_float(go0), __uint_as_float(go1)), bo);
    const float2 i_a = make_float2(p_sat_fma(pi.x, 0.2f, 0.5f), p_sat_fma(pi.y, 0.2f, 0.5f));
    const float2 f_a = make_float2(p_sat_fma(pf.x, 0.2f, 0.5f), p_sat_fma(pf.y, 0.2f, 0.5f));
    const float2 o_a = make_float2(p_sat_fma(po.x, 0.2f, 0.5f), p_sat_fma(po.y, 0.2f, 0.5f));
    const float2 g_a = make_float2(fmaxf(-1.f, fminf(1.f, pg.x)), fmaxf(-1.f, fminf(1.f, pg.y)));
    c = fma2(f_a, c, mul2(i_a, g_a));
    // exp(2c) = 2^(c * 2 log2 e)
    const float2 t = mul2(c, make_float2(2.885390043f, 2.885390043f));
    float ex, ey;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(t.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ey) : "f"(t.y));
    const float2 den = add2(make_float2(ex, ey), make_float2(1.f, 1.f));
    const float2 q = make_float2(__fdividef(2.0f, den.x), __fdividef(2.0f, den.y));
    const float2 th = add2(make_float2(1.f, 1.f), make_float2(-q.x, -q.y));
    const float2 hs = mul2(mul2(o_a, th), make_float2(127.f, 127.f));
    // round half away from zero: add 0.5 with the sign of the value, then truncate
    // (__fadd_rn: never fused with the multiplication before it)
    const float hx = __fadd_rn(hs.x, __uint_as_float(0x3F000000u | (__float_as_uint(hs.x) & 0x80000000u)));
    const float hy = __fadd_rn(hs.y, __uint_as_float(0x3F000000u | (__float_as_uint(hs.y) & 0x80000000u)));
    return (uint32_t(__float2int_rz(hx)) & 0xFFu) | ((uint32_t(__float2int_rz(hy)) & 0xFFu) << 8);
}

template <int UNITS, int WPT>
__global__ void __launch_bounds__(kPThreads, 1)
lstm_persist_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                    const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_w3,
                    const __grid_constant__ CUtensorMap tm_x,    // x_down  [T,B,R] f16
                    const __grid_constant__ CUtensorMap tm_hh,   // hh_down [1,B,R] f16
                    const __grid_constant__ CUtensorMap tm_dn,   // dn_hh   [R,H]   int8
                    const __grid_constant__ CUtensorMap tm_h,    // h_out   [T,B,H] int8
                    const __grid_constant__ CUtensorMap tm_h0,   // h_0     [1,B,H] int8
                    const __grid_constant__ CUtensorMap tm_hh_st,  // hh_down, boxes of a worker's 64 rows
                    const PersistDev p) {
    using L = PersistSmem<UNITS, WPT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
    uint64_t *bar_once = &bars[0];       // resident weights loaded
    uint64_t *bar_acc_full = &bars[1];   // [2] MMAs of the tile's step finished
    uint64_t *bar_acc_empty = &bars[3];  // [2] epilogue finished reading the accumulator
    uint64_t *bar_x = &bars[5];          // [2] gate: x_down tile filled
    uint64_t *bar_ahh = &bars[7];        // [2] gate: hh_down tile filled
    uint64_t *bar_epi = &bars[9];        // [2] epilogue warps have stored their part of the step
    uint64_t *bar_h = &bars[11];         // worker: its rows of the h tile filled
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kOffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_gate = p.n_pairs * p.n_slices;
    const bool is_gate = int(blockIdx.x) < n_gate;
    unsigned int *g_abort = p.flags + 2 * p.n_tiles;

    if (threadIdx.x == 0) {
        mbar_init(bar_once, 1);
        for (int g = 0; g < 2; ++g) {
            mbar_init(&bar_acc_full[g], 1);
            mbar_init(&bar_acc_empty[g], (is_gate || WPT == 2) ? 4 : 8);
            mbar_init(&bar_x[g], 1);
            mbar_init(&bar_ahh[g], 1);
            mbar_init(&bar_epi[g], (is_gate || WPT == 2) ? 4 : 8);
        }
        mbar_init(bar_h, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, L::kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    auto time_of = [&](int i) { return p.reverse ? p.T - 1 - i : i; };

    if (is_gate) {
        const int pair = blockIdx.x / p.n_slices;
        const int n0 = (blockIdx.x % p.n_slices) * UNITS;
        const int n_local = (2 * pair + 1 < p.n_tiles) ? 2 : 1;  // tiles this CTA really has
        if (warp == 0) {
            // ------------------------------ gate: producer ------------------------------
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_once, 4 * L::kWKB);
                for (int kb = 0; kb < 4; ++kb) {
                    uint8_t *sw = smem + L::kOffW + kb * L::kWKB;
                    tma_load_2d(sw + 0 * UNITS * 128, &tm_w0, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 1 * UNITS * 128, &tm_w1, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 2 * UNITS * 128, &tm_w2, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 3 * UNITS * 128, &tm_w3, bar_once, kb * 64, n0);
                }
                bool ok = true;
                for (int i = 0; i < p.T && ok; ++i) {
                    for (int g = 0; g < n_local && ok; ++g) {
                        const int m0 = (2 * pair + g) * 128;
                        // MMAs of the tile's previous step are done: both operand buffers are free
                        if (i > 0) ok = mbar_wait(&bar_acc_full[g], (i - 1) & 1, abort_flag, 32);
                        if (!ok) break;
                        uint8_t *sx = smem + L::kOffX + g * 32768;
                        mbar_arrive_expect_tx(&bar_x[g], 32768);
                        tma_load_4d(sx, &tm_x, &bar_x[g], 0, m0, 0, time_of(i));  // both K blocks
                    }
                    for (int g = 0; g < n_local && ok; ++g) {
                        const int tile = 2 * pair + g;
                        ok = wait_counter(p.flags + p.n_tiles + tile, (unsigned)(WPT * (i + 1)),
                                          g_abort, abort_flag, 33);
                        if (!ok) break;
                        FLUKE_STAMP(blockIdx.x == 0 && g == 0, i * 8 + 0, clock64());
                        fence_proxy_async_all();
                        uint8_t *sa = smem + L::kOffAhh + g * 32768;
                        mbar_arrive_expect_tx(&bar_ahh[g], 32768);
                        tma_load_3d(sa, &tm_hh, &bar_ahh[g], 0, tile * 128, 0);  // both K blocks
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ------------------------------ gate: MMA issuer ----------------------------
            constexpr uint32_t kIdesc = make_idesc<kKindF16>(128, 4 * UNITS);
            bool ok = mbar_wait(bar_once, 0, abort_flag, 34);
            for (int i = 0; i < p.T && ok; ++i) {
                for (int g = 0; g < n_local && ok; ++g) {  // x_down halves: W K blocks 2, 3
                    if (i > 0) ok = mbar_wait(&bar_acc_empty[g], (i - 1) & 1, abort_flag, 35);
                    if (!ok) break;
                    ok = mbar_wait(&bar_x[g], i & 1, abort_flag, 36);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint8_t *sx = smem + L::kOffX + g * 32768;
                        for (int kb = 0; kb < 2; ++kb) {
                            const uint64_t ad = make_smem_desc_sw128(smem_u32(sx + kb * 16384));
                            const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffW + (2 + kb) * L::kWKB));
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                tc_mma<kKindF16>(tmem_base + g * L::kAccStride, ad + uint64_t(2 * k),
                                                 bd + uint64_t(2 * k), kIdesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    __syncwarp();
                }
                for (int g = 0; g < n_local && ok; ++g) {  // hh_down halves: W K blocks 0, 1
                    ok = mbar_wait(&bar_ahh[g], i & 1, abort_flag, 37);
                    if (!ok) break;
                    FLUKE_STAMP(blockIdx.x == 0 && g == 0 && lane == 0, i * 8 + 1, clock64());
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint8_t *sa = smem + L::kOffAhh + g * 32768;
                        for (int kb = 0; kb < 2; ++kb) {
                            const uint64_t ad = make_smem_desc_sw128(smem_u32(sa + kb * 16384));
                            const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffW + kb * L::kWKB));
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                tc_mma<kKindF16>(tmem_base + g * L::kAccStride, ad + uint64_t(2 * k),
                                                 bd + uint64_t(2 * k), kIdesc, 1u);
                        }
                        tc_commit(&bar_acc_full[g]);
                    }
                    __syncwarp();
                }
            }
        } else {
            // ------------------------------ gate: epilogue ------------------------------
            const int g = (warp - 2) >> 2;  // which tile of the pair this warp set serves
            const int q = warp & 3;
            const int tile = 2 * pair + g;
            // stage the slice's biases in shared memory (read by every thread each step)
            float *sbias = reinterpret_cast<float *>(smem + L::kOffBias);
            for (int j = threadIdx.x - 64; j < 4 * UNITS; j += 256)
                sbias[j] = __ldg(p.bias + (j / UNITS) * p.H + n0 + (j % UNITS));
            asm volatile("bar.sync 2, 256;" ::: "memory");  // the eight epilogue warps, once, before any wait
            if (g < n_local) {
                const int row = tile * 128 + q * 32 + lane;
                const bool row_ok = row < p.B;
                float2 c2[UNITS / 2];  // the cell state of the slice, as pairs of adjacent units
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < UNITS / 4; ++v) {
                        const float4 c4 = *reinterpret_cast<const float4 *>(p.c + int64_t(row) * p.H + n0 + 4 * v);
                        c2[2 * v] = make_float2(c4.x, c4.y);
                        c2[2 * v + 1] = make_float2(c4.z, c4.w);
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < UNITS / 2; ++v) c2[v] = make_float2(0.f, 0.f);
                }
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + g * L::kAccStride;
                unsigned int *h_ready = p.flags + tile;
                bool ok = true;
                for (int i = 0; i < p.T && ok; ++i) {
                    ok = mbar_wait(&bar_acc_full[g], i & 1, abort_flag, 38);
                    if (!ok) break;
                    FLUKE_STAMP(blockIdx.x == 0 && threadIdx.x == 64, i * 8 + 2, clock64());
                    tc_fence_after_sync();
                    int8_t *hrow = p.h_out + (int64_t(time_of(i)) * p.b_stride + row) * p.H + n0;
#pragma unroll
                    for (int ch = 0; ch < UNITS / 8; ++ch) {
                        uint32_t gi[8], gf[8], gg[8], go[8];
                        tmem_ld_32x8(t_row + 0 * UNITS + ch * 8, gi);
                        tmem_ld_32x8(t_row + 1 * UNITS + ch * 8, gf);
                        tmem_ld_32x8(t_row + 2 * UNITS + ch * 8, gg);
                        tmem_ld_32x8(t_row + 3 * UNITS + ch * 8, go);
                        tmem_ld_wait();
                        if (ch == UNITS / 8 - 1) {
                            // all TMEM reads of this step are done: the next step's MMAs may overwrite
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&bar_acc_empty[g]);
                        }
                        uint32_t packed[2] = {0u, 0u};
#pragma unroll
                        for (int v = 0; v < 2; ++v) {
                            const int u = ch * 8 + 4 * v;
                            const float4 bi = *reinterpret_cast<const float4 *>(sbias + 0 * UNITS + u);
                            const float4 bf = *reinterpret_cast<const float4 *>(sbias + 1 * UNITS + u);
                            const float4 bg = *reinterpret_cast<const float4 *>(sbias + 2 * UNITS + u);
                            const float4 bo = *reinterpret_cast<const float4 *>(sbias + 3 * UNITS + u);
                            const int e = 4 * v;
                            const uint32_t lo = lstm_cell_pair(gi[e], gi[e + 1], gf[e], gf[e + 1], gg[e], gg[e + 1], go[e], go[e + 1],
                                                               make_float2(bi.x, bi.y), make_float2(bf.x, bf.y),
                                                               make_float2(bg.x, bg.y), make_float2(bo.x, bo.y), c2[(u >> 1)]);
                            const uint32_t hi = lstm_cell_pair(gi[e + 2], gi[e + 3], gf[e + 2], gf[e + 3], gg[e + 2], gg[e + 3],
                                                               go[e + 2], go[e + 3], make_float2(bi.z, bi.w), make_float2(bf.z, bf.w),
                                                               make_float2(bg.z, bg.w), make_float2(bo.z, bo.w), c2[(u >> 1) + 1]);
                            packed[v] = lo | (hi << 16);
                        }
                        if (row_ok) *reinterpret_cast<uint2 *>(hrow + ch * 8) = make_uint2(packed[0], packed[1]);
                    }
                    // publish this slice of h_t
                    ok = warps_barrier(&bar_epi[g], i & 1, lane, abort_flag);
                    if (ok && q == 2 && lane == 0) {
                        FLUKE_STAMP(blockIdx.x == 0 && g == 0, i * 8 + 3, clock64());
                        publish(h_ready);
                        FLUKE_STAMP(blockIdx.x == 0 && g == 0, i * 8 + 7, clock64());
                    }
                }
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < UNITS / 4; ++v)
                        *reinterpret_cast<float4 *>(p.c + int64_t(row) * p.H + n0 + 4 * v) =
                            make_float4(c2[2 * v].x, c2[2 * v].y, c2[2 * v + 1].x, c2[2 * v + 1].y);
                }
            }
        }
    } else {
        const int tile = (blockIdx.x - n_gate) / WPT;
        const int m0 = tile * 128 + ((blockIdx.x - n_gate) % WPT) * L::kWorkerRows;  // first row of this worker
        unsigned int *h_ready = p.flags + tile;
        unsigned int *hh_ready = p.flags + p.n_tiles + tile;
        if (warp == 0) {
            // ------------------------------ worker: producer ----------------------------
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_once, p.nkb_h * L::kDnKB);
                for (int kb = 0; kb < p.nkb_h; ++kb)
                    tma_load_2d(smem + L::kOffDn + kb * L::kDnKB, &tm_dn, bar_once, kb * 128, 0);
                bool ok = true;
                for (int i = 0; i < p.T && ok; ++i) {
                    if (i == 0 && (tile & 1)) {
                        // the second tile of a pair starts about half a step late and stays there:
                        // the two recurrences then use their gate CTA's epilogue warps' pipes (XU)
                        // alternately instead of at the same time
                        const long long t0 = clock64();
                        while (clock64() - t0 < kPStaggerCycles) {}
                    }
                    if (i > 0) {
                        ok = mbar_wait(&bar_acc_full[0], (i - 1) & 1, abort_flag, 48);  // h tile free again
                        if (!ok) break;
                        ok = wait_counter(h_ready, (unsigned)(p.n_slices * i), g_abort, abort_flag, 49);
                        if (!ok) break;
                        FLUKE_STAMP(int(blockIdx.x) == n_gate, i * 8 + 4, clock64());
                        fence_proxy_async_all();
                    }
                    // ONE instruction for the worker's rows of the whole tile: the map walks the K
                    // blocks of a row as its third dimension, so they land block after block (several
                    // smaller loads, which would let the contraction start earlier, measured slower)
                    mbar_arrive_expect_tx(bar_h, p.nkb_h * L::kHKB);
                    if (i == 0) tma_load_4d(smem + L::kOffH, &tm_h0, bar_h, 0, m0, 0, 0);
                    else tma_load_4d(smem + L::kOffH, &tm_h, bar_h, 0, m0, 0, time_of(i - 1));
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ------------------------------ worker: MMA issuer --------------------------
            constexpr uint32_t kIdesc = make_idesc<kKindI8>(128, kPRank);
            if (lane == 0) {
                bool ok = mbar_wait(bar_once, 0, abort_flag, 50);
                for (int i = 0; i < p.T && ok; ++i) {
                    if (i > 0) ok = mbar_wait(&bar_acc_empty[0], (i - 1) & 1, abort_flag, 51);
                    if (!ok) break;
                    ok = mbar_wait(bar_h, i & 1, abort_flag, 52);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (int kb = 0; kb < p.nkb_h; ++kb) {
                        // WPT == 2: rows 64-127 of the operand overlap the next K block (or the slack)
                        const uint64_t ad = make_smem_desc_sw128(smem_u32(smem + L::kOffH + kb * L::kHKB));
                        const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffDn + kb * L::kDnKB));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc_mma<kKindI8>(tmem_base, ad + uint64_t(2 * k), bd + uint64_t(2 * k), kIdesc,
                                            (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(&bar_acc_full[0]);
                }
            }
            __syncwarp();
        } else {
            // ------------------------------ worker: epilogue ----------------------------
            // The valid accumulator rows are TMEM lanes 0 .. kWorkerRows-1: with two workers per tile
            // only the warps of lane quadrants 0 and 1 take part (two per quadrant, 64 projection
            // columns each).
            const int q = warp & 3;
            if (q * 32 < L::kWorkerRows) {
                const int chalf = (warp - 2) >> 2;
                const int col0 = chalf * 64;
                float sc[64];
#pragma unroll
                for (int v = 0; v < 16; ++v) {
                    const float4 s4 = __ldg(reinterpret_cast<const float4 *>(p.dn_scale + col0) + v);
                    // same operand order as the dequant GEMM epilogue: sa * sb
                    sc[4 * v] = (1.0f / 127.0f) * s4.x; sc[4 * v + 1] = (1.0f / 127.0f) * s4.y;
                    sc[4 * v + 2] = (1.0f / 127.0f) * s4.z; sc[4 * v + 3] = (1.0f / 127.0f) * s4.w;
                }
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + col0;
                // The rows leave through shared memory and ONE bulk tensor store: a thread owns a
                // row, so direct stores would be 32 separate 16-byte pieces per instruction. The
                // staging tile is two blocks (column halves) of 64 rows x 128 bytes in the 128-byte
                // swizzle, which also makes the 16-byte writes of a warp conflict-free.
                const int srow = q * 32 + lane;
                uint8_t *stage_row = smem + L::kOffStage + chalf * (L::kStageBytes / 2) + srow * 128;
                bool ok = true;
                for (int i = 0; i < p.T && ok; ++i) {
                    ok = mbar_wait(&bar_acc_full[0], i & 1, abort_flag, 53);
                    if (!ok) break;
                    FLUKE_STAMP(int(blockIdx.x) == n_gate && threadIdx.x == 128, i * 8 + 5, clock64());
                    tc_fence_after_sync();
                    uint32_t acc0[32], acc1[32];
                    tmem_ld_32x32(t_row, acc0);
                    tmem_ld_32x32(t_row + 32, acc1);
                    tmem_ld_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_acc_empty[0]);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int e = (8 * v + 2 * j) & 31;
                            const uint32_t a0 = v < 4 ? acc0[e] : acc1[e];
                            const uint32_t a1 = v < 4 ? acc0[e + 1] : acc1[e + 1];
                            const __half2 h2 = __floats2half2_rn(float(int(a0)) * sc[8 * v + 2 * j],
                                                                 float(int(a1)) * sc[8 * v + 2 * j + 1]);
                            w[j] = *reinterpret_cast<const uint32_t *>(&h2);
                        }
                        *reinterpret_cast<uint4 *>(stage_row + ((v ^ (srow & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    fence_proxy_async_smem();
                    ok = warps_barrier(&bar_epi[0], i & 1, lane, abort_flag);
                    if (ok && warp == 4 && lane == 0) {
                        // rows past the end of the batch are clipped by the store
                        tma_store_3d(&tm_hh_st, smem + L::kOffStage, 0, m0, 0);
                        tma_store_commit();
                        tma_store_wait_all<0>();
                        publish(hh_ready);
                        FLUKE_STAMP(int(blockIdx.x) == n_gate, i * 8 + 6, clock64());
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

template <int UNITS, int WPT>
int persist_launch(const fluke_flstm_layer_t *l, const __half *x_down, __half *hh_down,
                   unsigned int *flags, int b0, int nb, cudaStream_t stream) {
    // one launch handles chunks [b0, b0+nb); all pointers below are offset to that range
    const int T = l->T, H = l->H, R = l->R, Bfull = l->B;
    auto kernel = lstm_persist_kernel<UNITS, WPT>;
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             PersistSmem<UNITS, WPT>::kDynamic);
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    PersistDev p;
    p.T = T; p.B = nb; p.b_stride = Bfull; p.H = H; p.reverse = l->reverse;
    p.n_tiles = (nb + 127) / 128; p.n_pairs = (p.n_tiles + 1) / 2;
    p.n_slices = H / UNITS; p.nkb_h = H / 128;
    p.bias = static_cast<const float *>(l->bias_f32);
    p.dn_scale = static_cast<const float *>(l->dn_hh_scale);
    p.c = static_cast<float *>(l->c_f32) + size_t(b0) * H;
    p.h_out = static_cast<int8_t *>(l->h_out_i8) + size_t(b0) * H;
    p.hh_down = hh_down + size_t(b0) * R;
    p.flags = flags;
    p.trace = trace_buffer();

    CUtensorMap tm_w[4], tm_x, tm_hh, tm_dn, tm_h, tm_h0, tm_hh_st;
    int rc;
    for (int g = 0; g < 4; ++g) {
        const __half *w = static_cast<const __half *>(l->w_up_f16) + size_t(g) * H * 2 * R;
        rc = make_tmap_2d(&tm_w[g], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w, H, 2 * R, uint64_t(2 * R) * 2, UNITS, 64, true);
        if (rc) return rc;
    }
    // planes are strided by the FULL batch; the row extent is this launch's nb rows
    // operand tiles come in with ONE instruction each: the maps walk the 128-byte K blocks of a
    // row as a dimension of their own (stride 128 bytes) outside the rows, so a box holds the
    // tile's K blocks one after the other, each in the 128-byte swizzle
    {
        const uint64_t dims[4] = {64, uint64_t(nb), 2, uint64_t(T)};
        const uint64_t strides[3] = {uint64_t(R) * 2, 128, uint64_t(Bfull) * R * 2};
        const uint32_t box[4] = {64, 128, 2, 1};
        rc = make_tmap_nd(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x_down + size_t(b0) * R, 4, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = make_tmap_nd(&tm_hh, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.hh_down, 3, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        const uint32_t box_st[3] = {64, 128 / WPT, 2};  // a worker's rows of a row tile
        rc = make_tmap_nd(&tm_hh_st, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.hh_down, 3, dims, strides, box_st,
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    rc = make_tmap_2d(&tm_dn, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, l->dn_hh_i8, R, H, H, kPRank, 128, true);
    if (rc) return rc;
    // the workers' maps: boxes of a worker's rows (half a row tile, or all of it) x all K blocks
    {
        const uint64_t dims[4] = {128, uint64_t(nb), uint64_t(p.nkb_h), uint64_t(T)};
        const uint64_t strides[3] = {uint64_t(H), 128, uint64_t(Bfull) * H};
        const uint32_t box[4] = {128, 128 / WPT, uint32_t(p.nkb_h), 1};
        rc = make_tmap_nd(&tm_h, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.h_out, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        const uint64_t dims0[4] = {128, uint64_t(nb), uint64_t(p.nkb_h), 1};
        rc = make_tmap_nd(&tm_h0, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<const int8_t *>(l->h_i8) + size_t(b0) * H, 4,
                          dims0, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }

    const int grid = p.n_pairs * p.n_slices + p.n_tiles * WPT;
    rc = (int)cudaMemsetAsync(flags, 0, sizeof(unsigned int) * (2 * p.n_tiles + 1), stream);
    if (rc) return rc;
    void *args[] = {&tm_w[0], &tm_w[1], &tm_w[2], &tm_w[3], &tm_x, &tm_hh, &tm_dn, &tm_h, &tm_h0, &tm_hh_st, &p};
    return (int)cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), dim3(grid), dim3(kPThreads),
                                            args, PersistSmem<UNITS, WPT>::kDynamic, stream);
}

// Largest number of 128-row tiles whose CTAs are all co-resident, or 0 when the device cannot
// run the kernel cooperatively.
template <int UNITS, int WPT>
int persist_max_tiles(int H) {
    int dev = 0, sms = 0, per_sm = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    auto kernel = lstm_persist_kernel<UNITS, WPT>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistSmem<UNITS, WPT>::kDynamic) != cudaSuccess)
        return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPThreads, PersistSmem<UNITS, WPT>::kDynamic) != cudaSuccess)
        return 0;
    if (!coop || per_sm < 1) return 0;
    const int slots = sms * per_sm, slices = H / UNITS;
    int tiles = 0;
    while (((tiles + 2) / 2) * slices + (tiles + 1) * WPT <= slots) ++tiles;
    return tiles;
}

}  // namespace
}  // namespace fluke_sm100

#ifdef FLUKE_SM100_TRACE
extern "C" void fluke_sm100_lstm_set_trace(void *device_buffer) {
    fluke_sm100::g_persist_trace = static_cast<long long *>(device_buffer);
}
#endif

// -1: the wide configuration (48 units per gate CTA, one worker per row tile: twice the row tiles
// per launch) is used when the layer has more row tiles than one launch of the narrow one holds;
// 0: never; 1: whenever the shape allows it.
static thread_local int g_lstm_wide = -1;  // per host thread, like the form selection
extern "C" void fluke_sm100_set_lstm_wide(int mode) { g_lstm_wide = mode < 0 ? -1 : (mode > 0 ? 1 : 0); }

// Runs the recurrence of one layer (x_down already computed) with persistent launches. Returns
// -2 when the shape is not covered (the caller then uses the per-step kernels).
extern "C" int fluke_sm100_lstm_layer_persistent(const void *layer, const void *x_down, void *hh_down,
                                                 void *flags, void *stream_) {
    using namespace fluke_sm100;
    const fluke_flstm_layer_t *l = static_cast<const fluke_flstm_layer_t *>(layer);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (l->R != kPRank || l->H % 128 || l->H > 128 * kPMaxHKB) return -2;
    const __half *xd = static_cast<const __half *>(x_down);
    __half *hd = static_cast<__half *>(hh_down);
    unsigned int *fl = static_cast<unsigned int *>(flags);
    // narrow configuration: hidden units per gate CTA 24 where H allows it (H = 768 -> 32 slices),
    // else 32; two workers per row tile
    const int units = (l->H % 24 == 0) ? 24 : 32;
    const int narrow_tiles = units == 24 ? persist_max_tiles<24, 2>(l->H) : persist_max_tiles<32, 2>(l->H);
    // wide configuration: 48 units per gate CTA, one worker per row tile
    const bool wide_ok = l->H % 48 == 0 && l->H <= 128 * PersistSmem<48, 1>::kMaxHKB;
    const int wide_tiles = wide_ok ? persist_max_tiles<48, 1>(l->H) : 0;
    const int tiles = (l->B + 127) / 128;
    const bool wide = wide_tiles > 0 && (g_lstm_wide == 1 || narrow_tiles < 1 ||
                                         (g_lstm_wide == -1 && tiles > narrow_tiles && wide_tiles > narrow_tiles));
    const int max_tiles = wide ? wide_tiles : narrow_tiles;
    if (max_tiles < 1) return -2;
    const int tiles_per_launch = max_tiles > 64 ? 64 : max_tiles;  // the counter block holds 2*64+1 words
    for (int b0 = 0; b0 < l->B; b0 += tiles_per_launch * 128) {
        const int nb = l->B - b0 < tiles_per_launch * 128 ? l->B - b0 : tiles_per_launch * 128;
        const int rc = wide ? persist_launch<48, 1>(l, xd, hd, fl, b0, nb, stream)
                            : (units == 24 ? persist_launch<24, 2>(l, xd, hd, fl, b0, nb, stream)
                                           : persist_launch<32, 2>(l, xd, hd, fl, b0, nb, stream));
        if (rc) return rc;
    }
    return 0;
}
