// Dense fp8 GEMM for the fully-connected / QKV / out / MLP projections on sm_100a:
//
//     out[M,N] = epilogue( (A[M,K] . W[N,K]^T) * (dq_a * dq_w) + bias[N] )
//
// A and W are fp8 codes (e4m3 or e5m2, independently), both K-contiguous ("TN"), which is the
// layout of upstream's FullyConnectedLayer: input [N_batch, in] and weights [out, in]
// (dnn/layers/fully_connected_layer.cu:15-41, launch :199-208).  This kernel replaces that launch.
//
// Structure: persistent CTAs (one per SM) loop over 128 x BN output tiles.
//   warp 0     TMA producer: 128-byte-swizzled K-blocks of A and W into a STAGES-deep smem ring
//   warp 1     MMA issuer:   tcgen05.mma kind::f8f6f4 (M=128, N=BN, K=32 per instruction),
//                            fp32 accumulators in TMEM, double-buffered (2 x BN columns)
//   warps 2..  epilogue:     fused dequant scale, bias, GELU (upstream activation_layer.cu:9-20 formula),
//                            residual add (upstream tensor.cu:383-415) and |out| max reduction.
//                            fp32 output: two warps per TMEM lane quarter, each taking every other 32-column
//                            chunk (the next chunk's tcgen05.ld in flight while this one is stored), through
//                            a per-warp smem transpose so that global stores are coalesced along N.
//                            fp8 output (32 codes = one 32-byte sector per thread and chunk) and the
//                            amax-only pass: four warps per quarter, all of a warp's chunks pulled into
//                            registers at once and the TMEM buffer handed back before any arithmetic.
// The epilogue of tile i overlaps the main loop of tile i+1 through the second TMEM buffer.
//
// Output modes: fp32 [M,N]; fp8 codes [M,N] quantised with a scale derived from a given max|out|;
// or nothing but max|out|.  df8_gemm_fp8_tn_q chains the last two (the GEMM runs twice) to produce
// per-tensor-quantised output without ever writing the fp32 tensor: at these K the second pass of
// tensor-core work is cheaper than 4+4+1 bytes per element of HBM round trip.
// All mbarrier waits are bounded; a wait that gives up records a code in the status word
// (df8_status_word_read) and the CTA tears down normally.
#include "df8_internal.cuh"
// mbarrier waits of the GEMM kernels sleep up to 1 ms per try (measured: 3.534 -> 3.510 ms per GPT-2 small forward,
// three runs each on one GPU; the attention kernels, whose waits are short and many, ran 1 % slower with it and
// keep the default)
#define DF8_MBAR_SUSPEND_NS 1000000
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

#include <atomic>
#include <cstdlib>

namespace df8 {

namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == fp8 elements per K-block (one 128-byte swizzle row)
constexpr int kEpiWarps = 8;
constexpr int kStagingFloatsPerWarp = 32 * 36;

// epilogue / output modes (template parameter MODE)
constexpr int kOutF32Vec = 0;   // fp32, N % 4 == 0 and 16-byte aligned pointers: 128-bit accesses
constexpr int kOutF32 = 1;      // fp32, any N
constexpr int kOutE4M3 = 2;     // fp8 codes, N % 16 == 0
constexpr int kOutE5M2 = 3;
constexpr int kOutNone = 4;     // max|out| only
constexpr int kOutF32Tma = 5;   // fp32 through TMA stores: row pitch a multiple of 4 floats, no residual, 256-column tiles
constexpr int kOutF32T = 6;     // fp32, TRANSPOSED: out[n * ldc + m], bias indexed by m (the skinny products of a decode step,
                                // computed as W . X^T so that the weight rows fill the 128-row tile)

// the modes whose epilogue works thread = row straight from registers (fp8 codes, max|out| only)
__host__ __device__ constexpr bool is_direct(int mode) { return mode == kOutE4M3 || mode == kOutE5M2 || mode == kOutNone; }

// Epilogue warps of the single-CTA kernel.  The fp32 modes are bound by their global stores and run two
// warps per TMEM lane quarter; the fp8 / amax-only modes are a chain of latencies (TMEM load, conversion,
// GELU) with nothing to store or little, and run four per quarter so that each SM sub-partition has four
// warps to interleave.
__host__ __device__ constexpr int epi_warps(int mode) { return is_direct(mode) ? 16 : 8; }
// per-warp staging bytes of the fp8 / amax modes: the bias slice (64 floats) and, for fp8 output, the codes tile
__host__ __device__ constexpr int direct_staging_bytes(int mode) { return mode == kOutNone ? 256 : 256 + 2048; }
__host__ __device__ constexpr int gemm_threads(int mode) { return 64 + 32 * epi_warps(mode); }

// Keep this struct at or below 128 bytes (a static_assert below checks it): above that size the compiler no longer
// scalarises the by-value kernel parameter but reads its fields through a register-held parameter address, and the
// kernels built that way raised an illegal memory access on a test shape (cause not established).  More per-launch
// data: a separate kernel parameter.
struct GemmArgs {
    const float* scale_a;   // {q, dq} of A
    const float* scale_w;   // {q, dq} of W
    const float* bias;      // [N] or null
    const float* residual;  // [M,N] or null
    float* out;             // [M,N] fp32 (fp32 modes)
    float* out_amax;        // 1 float or null
    uint8_t* out_codes;     // [M,N] fp8 codes (fp8 modes)
    const float* q_amax;    // max|out| the fp8 output scale is derived from (fp8 modes)
    float* out_scale;       // {q, dq} of the fp8 output, written by CTA 0 (fp8 modes), or null
    int M, N, K;
    int ldc;                // row pitch, in floats, of `out` and `residual` (fp32 modes)
    int a_slab_cols;        // A is stored as K / a_slab_cols row-major [M, a_slab_cols] slabs (K when it is one matrix)
    int flags;
    uint32_t idesc;
    unsigned int* status;
    unsigned int* grid_counter;  // fused max|out| + codes launch: arrival counter of the grid-wide barrier, else null
};

static_assert(sizeof(GemmArgs) <= 128, "GemmArgs must stay within 128 bytes: see the comment above the struct");

// Arrival counters of the fused launches' grid-wide barrier: each counts up for ever (a launch waits for the next
// multiple of its grid size), one of them per launch in turn so that launches that overlap in time do not mix.
// Every launch that uses them has one CTA per SM.
constexpr int kFusedCounters = 64;
__device__ unsigned int g_gemm_grid_counter[kFusedCounters] = {};

// TMA-store mode: two 128 x 32 fp32 boxes (16 KB each) per group of four epilogue warps, a 4 KB quarter per warp,
// then each warp's bias slice (its four chunks of a 256-column tile)
constexpr int kTmaBoxBytes = 32 * 32 * 4;
constexpr int kTmaBiasFloatsPerWarp = 128;
__host__ __device__ constexpr int tma_staging_bytes() { return kEpiWarps * (2 * kTmaBoxBytes + kTmaBiasFloatsPerWarp * 4); }

__host__ __device__ constexpr int pair_staging_bytes(int mode) {
    return mode == kOutF32Tma ? tma_staging_bytes()
           : mode == kOutF32T ? 0
           : is_direct(mode)  ? epi_warps(mode) * direct_staging_bytes(mode)
                              : kEpiWarps * kStagingFloatsPerWarp * 4;
}

template <int BN, int STAGES, int MODE>
struct GemmCfg {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // fp32 modes: a transpose buffer per epilogue warp; fp8 / amax modes: only each warp's bias slice
    static constexpr int kStagingBytes = pair_staging_bytes(MODE);
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kStagingBytes + kBarBytes + 1024;
    static constexpr int kTmemCols = 2 * BN;
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns: power of two");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void record_timeout(unsigned int* status, unsigned int code) {
    if (status) {
        atomicCAS(status, 0u, code);
        atomicAdd(status + 1, 1u);
    }
}

// x * 0.5 * (1 + tanh(0.7978845608 * (x + 0.044715 x^3))), evaluated as
//     u = x * fma(x*x, 0.7978845608*0.044715, 0.7978845608);   hx = 0.5 x;   gelu = fma(hx, tanh(u), hx)
// with explicit intrinsics (no compiler-chosen contraction), so that every epilogue variant produces identical
// bits; five arithmetic instructions and one tanh.approx per element (the fc1 epilogue is issue-bound).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float u = __fmul_rn(x, __fmaf_rn(__fmul_rn(x, x), 0.7978845608f * 0.044715f, 0.7978845608f));
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    const float hx = __fmul_rn(x, 0.5f);
    return __fmaf_rn(hx, t, hx);
}

// ---- fp32 output: transpose one 32-row x 32-column chunk through the warp's staging buffer -------

// thread = row: park the chunk's accumulators in shared memory
template <bool VEC4>
__device__ __forceinline__ void stage_chunk(const uint32_t (&r)[32], float* stg, int lane) {
    if constexpr (VEC4) {
        float4* srow = reinterpret_cast<float4*>(stg + lane * 36);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            srow[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
    } else {
        float* srow = stg + lane * 33;
#pragma unroll
        for (int j = 0; j < 32; ++j) srow[j] = __uint_as_float(r[j]);
    }
}

// The residual values a lane will add in store_chunk_f32<true> for the chunk at (row0, col0).  They do not depend
// on the accumulators, so the epilogue issues these loads one chunk ahead (for a tile's first chunk: before it
// waits for the MMAs) and their global-memory latency stays off the per-chunk chain.
__device__ __forceinline__ void load_residual_vec4(float4 (&rs)[8], int lane, int row0, int col0, const GemmArgs& a) {
    const int gcol = col0 + (lane & 7) * 4;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int rl = it * 4 + (lane >> 3);
        if ((a.flags & 2) && row0 + rl < a.M && gcol < a.N)
            rs[it] = __ldcg(reinterpret_cast<const float4*>(a.residual + size_t(row0 + rl) * a.ldc + gcol));
        else
            rs[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// lanes run along N: apply the epilogue and store coalesced.  `rs`: load_residual_vec4 of this chunk (VEC4 only).
template <bool VEC4>
__device__ __forceinline__ void store_chunk_f32(const float* stg, int lane, int row0, int col0, const GemmArgs& a,
                                                float alpha, float& amax, const float4 (&rs)[8]) {
    if constexpr (VEC4) {
        const int cq = (lane & 7) * 4;
        const int gcol = col0 + cq;
        const bool col_ok = gcol < a.N;
        // N need not be a multiple of 4 when the row pitch is: the last group of a row then hangs over N by up to
        // three columns, which land in the pitch padding; only the bias read and the maximum must stop at N
        const bool whole = gcol + 4 <= a.N;
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.bias && col_ok) {
            if (whole) {
                b4 = *reinterpret_cast<const float4*>(a.bias + gcol);
            } else {
                b4.x = a.bias[gcol];
                if (gcol + 1 < a.N) b4.y = a.bias[gcol + 1];
                if (gcol + 2 < a.N) b4.z = a.bias[gcol + 2];
            }
        }
        float4 v[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int rl = it * 4 + (lane >> 3);
            v[it] = *reinterpret_cast<const float4*>(stg + rl * 36 + cq);
        }
        // flag tests outside the per-element loops (a uniform branch per group costs more than the group's arithmetic)
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            v[it].x = fmaf(v[it].x, alpha, b4.x);
            v[it].y = fmaf(v[it].y, alpha, b4.y);
            v[it].z = fmaf(v[it].z, alpha, b4.z);
            v[it].w = fmaf(v[it].w, alpha, b4.w);
        }
        if (a.flags & 1) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                v[it].x = gelu_tanh(v[it].x);
                v[it].y = gelu_tanh(v[it].y);
                v[it].z = gelu_tanh(v[it].z);
                v[it].w = gelu_tanh(v[it].w);
            }
        }
        if (a.flags & 2) {  // not unconditionally: x + 0 would turn -0 into +0
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                v[it].x += rs[it].x;
                v[it].y += rs[it].y;
                v[it].z += rs[it].z;
                v[it].w += rs[it].w;
            }
        }
        if (col_ok) {
            const int row_first = row0 + (lane >> 3);
            if (a.flags & 4) {
                if (whole) {
#pragma unroll
                    for (int it = 0; it < 8; ++it)
                        if (row_first + it * 4 < a.M)
                            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[it].x), fabsf(v[it].y)), fmaxf(fabsf(v[it].z), fabsf(v[it].w))));
                } else {
#pragma unroll
                    for (int it = 0; it < 8; ++it)
                        if (row_first + it * 4 < a.M) {
                            amax = fmaxf(amax, fabsf(v[it].x));
                            if (gcol + 1 < a.N) amax = fmaxf(amax, fabsf(v[it].y));
                            if (gcol + 2 < a.N) amax = fmaxf(amax, fabsf(v[it].z));
                        }
                }
            }
            float* dst = a.out + size_t(row_first) * a.ldc + gcol;
            const size_t step = size_t(4) * a.ldc;
#pragma unroll
            for (int it = 0; it < 8; ++it)
                if (row_first + it * 4 < a.M) *reinterpret_cast<float4*>(dst + it * step) = v[it];
        }
    } else {
        // any N (e.g. a vocabulary of 50257): 4-byte accesses, a warp covers 128 contiguous bytes of one row;
        // the row pointer is advanced instead of recomputed and the row-tail test is hoisted
        const int gcol = col0 + lane;
        if (gcol < a.N) {
            const float b = a.bias ? a.bias[gcol] : 0.f;
            const int rows = min(32, a.M - row0);
            float* dst = a.out + size_t(row0) * a.ldc + gcol;
            const float* res = (a.flags & 2) ? a.residual + size_t(row0) * a.ldc + gcol : nullptr;
            const bool gelu = (a.flags & 1) != 0;
            if (rows == 32 && !res && !gelu) {
#pragma unroll
                for (int rl = 0; rl < 32; ++rl) {
                    const float v = fmaf(stg[rl * 33 + lane], alpha, b);
                    amax = fmaxf(amax, fabsf(v));
                    *dst = v;
                    dst += a.ldc;
                }
            } else {
                for (int rl = 0; rl < rows; ++rl) {
                    float v = fmaf(stg[rl * 33 + lane], alpha, b);
                    if (gelu) v = gelu_tanh(v);
                    if (res) {
                        v += __ldcg(res);
                        res += a.ldc;
                    }
                    amax = fmaxf(amax, fabsf(v));
                    *dst = v;
                    dst += a.ldc;
                }
            }
        }
    }
}

// ---- fp8 / amax-only output: thread = row, straight from registers ------------------------------

// KIND: DF8_E4M3 / DF8_E5M2 to emit codes, -1 to only reduce max|out|.
// `sbias`: the chunk's 32 bias values in shared memory (zeros without a bias), or null to read a.bias.
// Codes: the thread's 32 bytes (one row of the chunk) are parked as pieces 2j, 2j+1 of its row in the warp's
// staging tile `stg` ([32 rows][PP pieces of 16 bytes], pieces XOR-swizzled so that neither these writes nor the
// row-segment reads of store_staged_codes conflict); storing them from here, 16 bytes per row and instruction,
// cost 6-10 us per pass (measured): the stores must leave as whole row segments.
template <int KIND, int PP = 2>
__device__ __forceinline__ void direct_chunk(const uint32_t (&r)[32], int grow, int col0, const GemmArgs& a,
                                             float alpha, float out_q, float& amax, const float* sbias = nullptr,
                                             uint8_t* stg = nullptr, int j = 0) {
    const bool row_ok = grow < a.M;
    uint32_t w[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sbias) b4 = *reinterpret_cast<const float4*>(sbias + 4 * g);  // broadcast read
        else if (a.bias) b4 = __ldg(reinterpret_cast<const float4*>(a.bias + col0 + 4 * g));  // same address in every lane
        float v0 = fmaf(__uint_as_float(r[4 * g]), alpha, b4.x);
        float v1 = fmaf(__uint_as_float(r[4 * g + 1]), alpha, b4.y);
        float v2 = fmaf(__uint_as_float(r[4 * g + 2]), alpha, b4.z);
        float v3 = fmaf(__uint_as_float(r[4 * g + 3]), alpha, b4.w);
        if (a.flags & 1) {
            v0 = gelu_tanh(v0);
            v1 = gelu_tanh(v1);
            v2 = gelu_tanh(v2);
            v3 = gelu_tanh(v3);
        }
        if constexpr (KIND < 0) {
            if (row_ok) amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
        } else {
            w[g] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(v0, out_q), __fmul_rn(v1, out_q), __fmul_rn(v2, out_q),
                                            __fmul_rn(v3, out_q));
        }
    }
    if constexpr (KIND >= 0) {
        const int lane = threadIdx.x & 31;
        const int sw = PP == 4 ? ((lane >> 1) & 3) : ((lane >> 2) & 1);
        uint8_t* srow = stg + lane * (PP * 16);
        *reinterpret_cast<uint4*>(srow + (((2 * j) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(srow + (((2 * j + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    (void)row_ok;
}

// The warp's staged codes ([32 rows][PP x 16 bytes], columns col0 .. col0 + 16 PP) to global memory: PP lanes cover
// one row's contiguous PP x 16 bytes, 32 / PP rows per instruction.
template <int PP>
__device__ __forceinline__ void store_staged_codes(const uint8_t* stg, int lane, int row0, int col0, const GemmArgs& a) {
    constexpr int kRowsPerInstr = 32 / PP;
    const int p = lane % PP;
#pragma unroll
    for (int it = 0; it < PP; ++it) {
        const int rr = it * kRowsPerInstr + lane / PP;
        const int sw = PP == 4 ? ((rr >> 1) & 3) : ((rr >> 2) & 1);
        const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * (PP * 16) + ((p ^ sw) << 4));
        if (row0 + rr < a.M && col0 + 16 * p < a.N)
            *reinterpret_cast<uint4*>(a.out_codes + size_t(row0 + rr) * a.N + col0 + 16 * p) = v;
    }
}

// ---- fp32 output through TMA stores (kOutF32Tma) ----------------------------------------------------
//
// thread = row.  A 32 x 32 chunk is scaled, biased (and GELU'd) in registers and parked in shared memory in the
// 128-byte-swizzled layout of the output tensor map (16-byte piece c of row r at piece c ^ (r & 7): neither these
// writes nor the copy engine's reads conflict); a cp.async.bulk.tensor store then takes it to global memory while
// the warps work on the next chunk.  The store clips rows >= M and columns >= N itself, so edge tiles need no
// predication and the pitch padding of a row is never written.  Against the transpose through shared memory +
// 128-bit st.global of the other fp32 modes this takes the global stores (and the second pass over shared memory)
// off the warps: the vocabulary head, whose 1.6 GB of logits make the epilogue the longest phase of a tile, is the
// case it is for.
// ONE store per 128 x 32 piece of the tile: the four warps that share a chunk index (one per TMEM lane quarter)
// fill the four 4 KB quarters of one 16 KB box (the swizzle pattern repeats every 8 rows, so a quarter is laid out
// like a box of its own), meet at a named barrier, and warp 0 of the group issues the store.  Before it arrives at
// that barrier the issuing lane has waited for the group's previous store to be done READING its box, so every
// warp that leaves the barrier may fill the other box at once: one barrier per chunk.  `box_it` counts the group's
// stores over the whole kernel (box box_it & 1 is the next one to fill).  Returns false when the wait for the
// accumulators gave up.
// What the clock stamps of this epilogue showed on the vocabulary head (8192 x 50257 x 768, CTA pairs), and what
// the code keeps from them: (1) every flag test inside the per-element loops is a uniform branch that costs more
// than the arithmetic it guards (30 branches per chunk, ~1000 cycles against ~100 for the multiply-adds), so the
// flags are tested once per chunk around whole loops, here and in the other epilogues; (2) the bias values are
// read into registers in one go before the accumulators are waited for: read one by one between the stores they
// cannot be moved up by the compiler (the stores might alias them) and each costs a shared-memory round trip of
// ~150 cycles while the operand ring is busy; (3) the size of the store (4 KB per warp or 16 KB per group) made
// no difference to the head, 16 KB helps at K = 4096 (1570 -> 1390 us for 8192 x 50257 x 4096).
template <int BN, typename ReleaseFn>
__device__ __forceinline__ bool epilogue_tile_f32_tma_group(const CUtensorMap* tma_out, const GemmArgs& args,
                                                            uint8_t* group_boxes, float* sbias, uint32_t tfull_bar,
                                                            uint32_t acc_phase, uint32_t taddr, int tile_row0, int q,
                                                            int n0, int half, int lane, float alpha, float& amax,
                                                            uint32_t& box_it, ReleaseFn release) {
    constexpr int kChunks = BN / 64;
    static_assert(kChunks * 32 <= kTmaBiasFloatsPerWarp, "bias slice");
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        const int col = n0 + 32 * (half + 2 * j) + lane;
        sbias[j * 32 + lane] = (args.bias && col < args.N) ? __ldg(args.bias + col) : 0.f;
    }
    __syncwarp();
    if (!mbar_wait_bounded(tfull_bar, acc_phase)) return false;
    tc_fence_after_sync();
    int nvalid = 0;  // the same for the four warps of a group
#pragma unroll
    for (int j = 0; j < kChunks; ++j)
        if (n0 + 32 * (half + 2 * j) < args.N) nvalid = j + 1;
    uint32_t r[32];
    if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, r);
    const bool row_ok = tile_row0 + q * 32 + lane < args.M;
    for (int j = 0; j < nvalid; ++j) {
        const int col0 = n0 + 32 * (half + 2 * j);
        uint8_t* box = group_boxes + (box_it & 1u) * (4 * kTmaBoxBytes);
        uint8_t* mine = box + q * kTmaBoxBytes;
        // the chunk's bias values, all eight reads in flight at once and before the accumulators are waited for:
        // read one by one between the stores below they cannot be moved up by the compiler (the stores might
        // alias them) and each costs a full shared-memory round trip, ~150 cycles while the operand ring is busy
        float4 bq[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) bq[g] = *reinterpret_cast<const float4*>(sbias + j * 32 + 4 * g);  // broadcast reads
        tmem_ld_wait();
        // flag tests stay outside the per-element loops: a uniform branch per four elements cost more than the
        // arithmetic (30 branches per chunk, ~1000 cycles against ~100 for the multiply-adds)
        float o[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            o[4 * g] = fmaf(__uint_as_float(r[4 * g]), alpha, bq[g].x);
            o[4 * g + 1] = fmaf(__uint_as_float(r[4 * g + 1]), alpha, bq[g].y);
            o[4 * g + 2] = fmaf(__uint_as_float(r[4 * g + 2]), alpha, bq[g].z);
            o[4 * g + 3] = fmaf(__uint_as_float(r[4 * g + 3]), alpha, bq[g].w);
        }
        if (args.flags & 1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = gelu_tanh(o[i]);
        }
        if ((args.flags & 4) && row_ok) {
            if (col0 + 32 <= args.N) {
                float m0 = 0.f, m1 = 0.f;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    m0 = fmaxf(m0, fabsf(o[i]));
                    m1 = fmaxf(m1, fabsf(o[i + 1]));
                }
                amax = fmaxf(amax, fmaxf(m0, m1));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < args.N) amax = fmaxf(amax, fabsf(o[i]));
            }
        }
#pragma unroll
        for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(mine + lane * 128 + ((g ^ (lane & 7)) << 4)) =
                make_float4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]);
        fence_proxy_async_smem();  // each lane's writes become visible to the copy engine
        if (j + 1 < nvalid) {
            tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), r);  // in flight across the barrier and the store
        } else {
            tc_fence_before_sync();  // the tile's last chunk is out of TMEM: hand the buffer back
            __syncwarp();
            release();
        }
        // the other box (filled next) was read by the store before last; the issuing lane alone knows its bulk groups
        if (q == 0 && lane == 0) tma_store_wait_read<0>();
        asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
        if (q == 0 && lane == 0) {
            tma_store_2d(tma_out, smem_u32(box), col0, tile_row0);
            tma_store_commit();
        }

        ++box_it;
    }
    if (nvalid == 0) {
        tc_fence_before_sync();
        __syncwarp();
        release();
    }
    return true;
}

// ---- fp32 output, transposed (kOutF32T) ------------------------------------------------------------------
//
// A decode step multiplies a handful of token rows (the batch) with a whole weight matrix: the product is bound by
// streaming the weights from HBM, and with the tokens as the M dimension a 128-row tile would be almost empty.  So
// the operands swap roles: the kernel's A is the WEIGHT matrix [rows = output features, K] and its "W" operand the
// activations [batch, K]; the accumulator tile is [128 features, batch] and leaves transposed, out[b * ldc + f].
// thread = feature row, so for a fixed batch column the 32 lanes of a warp write 32 consecutive floats.  bias is
// indexed by the feature (row), the residual is read at the output's position.
// One chunk: this lane's feature row, 32 consecutive token columns col0 .. col0 + 31.  Flag tests stay outside the
// per-element loops (a uniform branch per element costs more than its arithmetic).
// The residual values of one chunk (this lane's feature row, token columns col0 .. col0 + 31), zero outside the
// output.  They do not depend on the accumulators: the epilogue asks for a chunk's values one chunk ahead (for a
// tile's first chunk before it waits for the MMAs), so their global-memory latency stays off the per-chunk chain.
__device__ __forceinline__ void load_residual_transposed(float (&rs)[32], const GemmArgs& args, int grow, bool row_ok, int col0) {
    const size_t ldc = size_t(args.ldc);
    const float* res = args.residual + size_t(col0) * ldc + grow;
    if (row_ok && col0 + 32 <= args.N) {
#pragma unroll
        for (int i = 0; i < 32; ++i) rs[i] = __ldcg(res + i * ldc);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) rs[i] = (row_ok && col0 + i < args.N) ? __ldcg(res + i * ldc) : 0.f;
    }
}

// `rs`: the chunk's residual values on entry; refilled with those of the chunk at next_col0 (>= 0) once they have been
// added, before the stores are issued.
__device__ __forceinline__ void store_chunk_transposed(const uint32_t (&r)[32], const GemmArgs& args, int grow, int col0,
                                                       float alpha, float b, float& amax, float (&rs)[32], int next_col0) {
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = fmaf(__uint_as_float(r[i]), alpha, b);
    if (args.flags & 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = gelu_tanh(o[i]);
    }
    if (args.flags & 2) {  // not unconditionally: x + 0 would turn -0 into +0
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] += rs[i];
        if (next_col0 >= 0) load_residual_transposed(rs, args, grow, true, next_col0);
    }
    const size_t ldc = size_t(args.ldc);
    float* dst = args.out + size_t(col0) * ldc + grow;
    if (col0 + 32 <= args.N) {
        if (args.flags & 4) {
            float m0 = 0.f, m1 = 0.f;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                m0 = fmaxf(m0, fabsf(o[i]));
                m1 = fmaxf(m1, fabsf(o[i + 1]));
            }
            amax = fmaxf(amax, fmaxf(m0, m1));
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[i * ldc] = o[i];
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (col0 + i < args.N) {
                if (args.flags & 4) amax = fmaxf(amax, fabsf(o[i]));
                dst[i * ldc] = o[i];
            }
        }
    }
}

template <int BN, typename ReleaseFn>
__device__ __forceinline__ bool epilogue_tile_f32_transposed(const GemmArgs& args, uint32_t tfull_bar, uint32_t acc_phase,
                                                             uint32_t taddr, int row0, int n0, int half, int lane,
                                                             float alpha, float& amax, ReleaseFn release) {
    constexpr int kChunks = BN / 64;  // this warp's chunks: half, half + 2, ...
    const int grow = row0 + lane;
    const bool row_ok = grow < args.M;
    const float b = (args.bias && row_ok) ? __ldg(args.bias + grow) : 0.f;
    const bool with_res = (args.flags & 2) != 0;
    float rs[32];
    if (with_res && n0 + 32 * half < args.N) load_residual_transposed(rs, args, grow, row_ok, n0 + 32 * half);
    if (!mbar_wait_bounded(tfull_bar, acc_phase)) return false;
    tc_fence_after_sync();
    int nvalid = 0;
#pragma unroll
    for (int j = 0; j < kChunks; ++j)
        if (n0 + 32 * (half + 2 * j) < args.N) nvalid = j + 1;
    // two register sets: the next chunk's accumulators are on their way while this one is stored
    uint32_t ra[32], rb[32];
    if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, ra);
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        if (j < nvalid) {
            tmem_ld_wait();
            if (j + 1 < nvalid) {
                if (j & 1) tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), ra);
                else tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), rb);
            } else {
                tc_fence_before_sync();
                __syncwarp();
                release();
            }
            if (row_ok) {
                const int next_col0 = (with_res && j + 1 < nvalid) ? n0 + 32 * (half + 2 * (j + 1)) : -1;
                if (j & 1) store_chunk_transposed(rb, args, grow, n0 + 32 * (half + 2 * j), alpha, b, amax, rs, next_col0);
                else store_chunk_transposed(ra, args, grow, n0 + 32 * (half + 2 * j), alpha, b, amax, rs, next_col0);
            }
        }
    }
    if (nvalid == 0) {
        tc_fence_before_sync();
        __syncwarp();
        release();
    }
    return true;
}

// FUSED (fp8 modes only): the one-launch max|out| + codes form, an instantiation of its own so that the plain
// kernels carry none of its code or registers.
template <int BN, int STAGES, int MODE, bool FUSED = false>
__global__ void __launch_bounds__(gemm_threads(MODE), 1)
gemm_fp8_tn_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_w,
                   const __grid_constant__ CUtensorMap tma_out, const GemmArgs args) {
    static_assert(!FUSED || MODE == kOutE4M3 || MODE == kOutE5M2, "the fused form emits fp8 codes");
    using Cfg = GemmCfg<BN, STAGES, MODE>;
    constexpr int EW = epi_warps(MODE);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* staging = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes + Cfg::kStagingBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tfull = bars + 2 * STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    griddep_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(tfull + b), 1);
            mbar_init(smem_u32(tempty + b), EW);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    griddep_wait();  // everything above overlaps the previous kernel's tail; global memory is touched below

    const int num_m = (args.M + BM - 1) / BM;
    const int num_n = (args.N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (args.K + BK - 1) / BK;
    // This CTA's tiles: blockIdx.x + k * gridDim.x, k < n_mine.  A fused launch (max|out|, grid-wide barrier, codes;
    // fp8 modes only) walks them twice, except that the accumulators of its last n_keep tiles stay in TMEM over the
    // barrier and are not computed again: the sequence is k = 0 .. n_mine-1, then 0 .. n_mine-n_keep-1.
    constexpr bool fused = FUSED;
    const int n_mine = int(blockIdx.x) < num_tiles ? (num_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const int n_keep = fused ? (n_mine < 2 ? n_mine : 2) : 0;
    const int seq_len = fused ? 2 * n_mine - n_keep : n_mine;
    auto seq_tile = [&](int i) { return int(blockIdx.x) + (i < n_mine ? i : i - n_mine) * int(gridDim.x); };

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tma_a);
            prefetch_tensormap(&tma_w);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            if constexpr (MODE == kOutF32Tma) prefetch_tensormap(&tma_out);
            for (int i = 0; i < seq_len && ok; ++i) {
                const int tile = seq_tile(i);
                const int m0 = (tile % num_m) * BM;
                const int n0 = (tile / num_m) * BN;
                int ax = 0, aslab = 0;  // A's K coordinate: column inside its slab, slab index
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(empty + stage), phase ^ 1)) {
                        record_timeout(args.status, 0x100u + stage);
                        ok = false;
                        break;
                    }
                    const uint32_t fb = smem_u32(full + stage);
                    uint8_t* sa = smem + stage * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(fb, Cfg::kStageBytes);
                    tma_load_3d(smem_u32(sa), &tma_a, fb, ax, m0, aslab);
                    tma_load_2d(smem_u32(sa + Cfg::kABytes), &tma_w, fb, kb * BK, n0);
                    ax += BK;
                    if (ax >= args.a_slab_cols) {
                        ax = 0;
                        ++aslab;
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // This thread's scalar instructions are the issue-rate limit at BN = 128 (a K block is consumed
            // in 256 cycles), so the loop carries ready-made values: the descriptor of the stage's A tile as
            // a 32-bit low half that steps with the ring, and the barrier addresses likewise.
            const uint64_t desc0 = make_desc_kmajor_sw128(smem_u32(smem));
            const uint32_t dhi = desc_hi(desc0), dlo0 = desc_lo(desc0);
            constexpr uint32_t kStageStep = Cfg::kStageBytes >> 4, kBOff = Cfg::kABytes >> 4;
            const uint32_t full0 = smem_u32(full), empty0 = smem_u32(empty);
            const uint32_t idesc = args.idesc;
            int stage = 0;
            uint32_t phase = 0, dlo = dlo0, fullb = full0, emptyb = empty0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int i = 0; i < seq_len && ok; ++i, ++acc_it) {
                const uint32_t buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                // (fused: the buffers of the kept tiles come back in the second phase, after their codes are out)
                if (!mbar_wait_bounded(smem_u32(tempty + buf), acc_phase ^ 1)) {
                    record_timeout(args.status, 0x200u + buf);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(fullb, phase)) {
                        record_timeout(args.status, 0x300u + stage);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t alo = dlo, blo = dlo + kBOff;
                    if (kb == 0) tc_mma_f8(d_tmem, desc_join(alo, dhi), desc_join(blo, dhi), idesc, 0);
                    else tc_mma_f8_acc(d_tmem, desc_join(alo, dhi), desc_join(blo, dhi), idesc);
#pragma unroll
                    for (int k = 1; k < BK / 32; ++k)  // 32 bytes of K = 2 descriptor address units
                        tc_mma_f8_acc(d_tmem, desc_join(alo + 2 * k, dhi), desc_join(blo + 2 * k, dhi), idesc);
                    tc_commit(emptyb);
                    dlo += kStageStep;
                    fullb += 8;
                    emptyb += 8;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                        dlo = dlo0;
                        fullb = full0;
                        emptyb = empty0;
                    }
                }
                if (ok) tc_commit(smem_u32(tfull + buf));
            }
        }
    } else {
        const int e = warp - 2;
        const int q = warp & 3;    // TMEM lane quarter this warp may read
        const int half = e >> 2;   // which of the quarter's two warps: takes chunks half, half+2, ...
        constexpr int kChunks = BN / 64;  // 32-column chunks per warp and tile
        float* stg = staging + e * kStagingFloatsPerWarp;
        const float alpha = ld_l2_f32(args.scale_a + 1) * ld_l2_f32(args.scale_w + 1);
        float out_q = 1.f;
        if constexpr (MODE == kOutE4M3 || MODE == kOutE5M2) {
            if (!fused) {
                const float2 sc = scales_from_amax(ld_l2_f32(args.q_amax), fp8_max(MODE == kOutE4M3 ? DF8_E4M3 : DF8_E5M2));
                out_q = sc.x;
                if (blockIdx.x == 0 && e == 0 && lane == 0 && args.out_scale) {
                    args.out_scale[0] = sc.x;
                    args.out_scale[1] = sc.y;
                }
            }
        }
        const uint32_t lane_addr = uint32_t(q * 32) << 16;
        uint32_t acc_it = 0;
        uint32_t box_it = 0;  // TMA-store mode: running count of this warp's stores (alternates its two boxes)
        float amax = 0.f;  // max|out| over all of this warp's tiles: one atomic per warp at the end
        if constexpr (MODE == kOutE4M3 || MODE == kOutE5M2) {
            if (fused) {
                constexpr int KIND = MODE == kOutE4M3 ? int(DF8_E4M3) : int(DF8_E5M2);
                constexpr int kParts = EW / 4;
                constexpr int kCh = BN / (32 * kParts);
                const int part = e >> 2;
                uint8_t* wst = reinterpret_cast<uint8_t*>(staging) + e * direct_staging_bytes(MODE);
                float* sb = reinterpret_cast<float*>(wst);
                uint8_t* codes_tile = wst + 256;
                bool ok = true;
                // One tile of the sequence: accumulators into registers (after waiting for the MMAs unless they were
                // kept from the first phase), TMEM handed back unless the tile is kept, then max|out| or codes.
                auto do_tile = [&](int k, uint32_t it, bool wait_full, bool release, bool codes) {
                    const int tile = int(blockIdx.x) + k * int(gridDim.x);
                    const uint32_t buf = it & 1;
                    const int m0 = (tile % num_m) * BM, n0 = (tile / num_m) * BN;
                    const int row0 = m0 + q * 32;
                    const uint32_t taddr = tmem_base + buf * BN + lane_addr;
                    const int colw = n0 + 32 * kCh * part;
#pragma unroll
                    for (int j = 0; j < kCh; ++j) {
                        const int col = colw + 32 * j + lane;
                        sb[j * 32 + lane] = (args.bias && col < args.N) ? __ldg(args.bias + col) : 0.f;
                    }
                    __syncwarp();
                    if (wait_full && ok && !mbar_wait_bounded(smem_u32(tfull + buf), (it >> 1) & 1)) {
                        if (lane == 0) record_timeout(args.status, 0x400u + buf);
                        ok = false;  // keep walking (the barriers below need every warp), without touching TMEM
                    }
                    uint32_t r[kCh][32];
                    if (ok) {
                        tc_fence_after_sync();
#pragma unroll
                        for (int j = 0; j < kCh; ++j)
                            if (colw + 32 * j < args.N) tmem_ld_32x32(taddr + 32 * (kCh * part + j), r[j]);
                        tmem_ld_wait();
                        tc_fence_before_sync();
                    }
                    __syncwarp();
                    if (release && lane == 0) mbar_arrive(smem_u32(tempty + buf));
                    if (ok) {
                        const int grow = row0 + lane;
#pragma unroll
                        for (int j = 0; j < kCh; ++j) {
                            const int col0 = colw + 32 * j;
                            if (col0 < args.N) {
                                if (codes) direct_chunk<KIND, 2 * kCh>(r[j], grow, col0, args, alpha, out_q, amax, sb + j * 32, codes_tile, j);
                                else direct_chunk<-1>(r[j], grow, col0, args, alpha, 1.f, amax, sb + j * 32);
                            }
                        }
                        __syncwarp();
                        if (codes) {
                            store_staged_codes<2 * kCh>(codes_tile, lane, row0, colw, args);
                            __syncwarp();
                        }
                    }
                };
                // phase 1: max|out| over every tile; the last n_keep tiles stay in TMEM
                for (int k = 0; k < n_mine; ++k) do_tile(k, uint32_t(k), true, k < n_mine - n_keep, false);
                amax = warp_max(amax);
                if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
                // grid-wide barrier (bounded): every CTA's maxima are in before anyone reads the result
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
                if (e == 0 && lane == 0) {
                    __threadfence();
                    const unsigned int ticket = atomicAdd(args.grid_counter, 1u);
                    const unsigned int target = (ticket / gridDim.x + 1u) * gridDim.x;
                    volatile unsigned int* cnt = args.grid_counter;
                    unsigned long long t0 = 0;
                    // (one poller per CTA, a quarter of a microsecond apart: 148 CTAs polling one address every few
                    // tens of nanoseconds would load its L2 slice with a few billion reads per second while the
                    // slower CTAs still stream operands)
                    for (unsigned int spins = 0; int(*cnt - target) < 0; ++spins) {
                        __nanosleep(256);
                        if ((spins & 1023u) == 1023u) {
                            const unsigned long long now = globaltimer_ns();
                            if (t0 == 0) t0 = now;
                            if (now - t0 > 2000000000ull) {  // a CTA never came: flag it and finish
                                record_timeout(args.status, 0x4800u);
                                break;
                            }
                        }
                    }
                    __threadfence();
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");
                {
                    const float2 sc = scales_from_amax(*reinterpret_cast<const volatile float*>(args.out_amax),
                                                       fp8_max(MODE == kOutE4M3 ? DF8_E4M3 : DF8_E5M2));
                    out_q = sc.x;
                    if (blockIdx.x == 0 && e == 0 && lane == 0 && args.out_scale) {
                        args.out_scale[0] = sc.x;
                        args.out_scale[1] = sc.y;
                    }
                }
                amax = 0.f;
                // phase 2: codes; first the kept tiles straight from TMEM, then the others as the MMAs redo them
                for (int k = n_mine - n_keep; k < n_mine; ++k) do_tile(k, uint32_t(k), false, true, true);
                for (int k = 0; k < n_mine - n_keep; ++k) do_tile(k, uint32_t(n_mine + k), true, true, true);
                acc_it = uint32_t(seq_len);
            }
        }
        for (int tile = blockIdx.x; tile < num_tiles && !fused; tile += gridDim.x, ++acc_it) {
            const uint32_t buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            const int m0 = (tile % num_m) * BM;
            const int n0 = (tile / num_m) * BN;
            const int row0 = m0 + q * 32;
            const uint32_t taddr = tmem_base + buf * BN + lane_addr;
            if constexpr (MODE == kOutF32T) {
                auto release = [&] {
                    if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                };
                if (!epilogue_tile_f32_transposed<BN>(args, smem_u32(tfull + buf), acc_phase, taddr, row0, n0, half, lane,
                                                      alpha, amax, release)) {
                    if (lane == 0) record_timeout(args.status, 0x400u + buf);
                    break;
                }
                continue;
            }
            if constexpr (MODE == kOutF32Tma) {
                uint8_t* group_boxes = reinterpret_cast<uint8_t*>(staging) + half * (8 * kTmaBoxBytes);
                float* sbias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(staging) + kEpiWarps * 2 * kTmaBoxBytes) +
                               e * kTmaBiasFloatsPerWarp;
                auto release = [&] {
                    if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                };
                const bool ok = epilogue_tile_f32_tma_group<BN>(&tma_out, args, group_boxes, sbias, smem_u32(tfull + buf), acc_phase,
                                                                taddr, m0, q, n0, half, lane, alpha, amax, box_it, release);
                if (!ok) {
                    if (lane == 0) record_timeout(args.status, 0x400u + buf);
                    break;
                }
                continue;
            }
            if constexpr (is_direct(MODE)) {
                // Four warps per lane quarter; warp `part` takes the 32-column chunks part, part + 4, ...
                // Its bias slice goes to shared memory before the accumulators are waited for; the chunks
                // are pulled into registers in one go and the TMEM buffer is handed back before any math.
                constexpr int KIND = MODE == kOutE4M3 ? int(DF8_E4M3) : (MODE == kOutE5M2 ? int(DF8_E5M2) : -1);
                constexpr int kParts = EW / 4;
                constexpr int kCh = BN / (32 * kParts);
                const int part = e >> 2;
                // this warp's columns: kCh adjacent chunks, so that its codes of a row are one contiguous segment
                const int colw = n0 + 32 * kCh * part;
                uint8_t* wst = reinterpret_cast<uint8_t*>(staging) + e * direct_staging_bytes(MODE);
                float* sb = reinterpret_cast<float*>(wst);
                uint8_t* codes_tile = wst + 256;
#pragma unroll
                for (int j = 0; j < kCh; ++j) {
                    const int col = colw + 32 * j + lane;
                    sb[j * 32 + lane] = (args.bias && col < args.N) ? __ldg(args.bias + col) : 0.f;
                }
                __syncwarp();
                if (!mbar_wait_bounded(smem_u32(tfull + buf), acc_phase)) {
                    if (lane == 0) record_timeout(args.status, 0x400u + buf);
                    break;
                }
                tc_fence_after_sync();
                uint32_t r[kCh][32];
#pragma unroll
                for (int j = 0; j < kCh; ++j)
                    if (colw + 32 * j < args.N) tmem_ld_32x32(taddr + 32 * (kCh * part + j), r[j]);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                const int grow = row0 + lane;
#pragma unroll
                for (int j = 0; j < kCh; ++j) {
                    const int col0 = colw + 32 * j;
                    if (col0 < args.N)
                        direct_chunk<KIND, 2 * kCh>(r[j], grow, col0, args, alpha, out_q, amax, sb + j * 32, codes_tile, j);
                }
                __syncwarp();  // the codes tile is complete (and every lane is done with the bias slice)
                if constexpr (KIND >= 0) {
                    store_staged_codes<2 * kCh>(codes_tile, lane, row0, colw, args);
                    __syncwarp();  // before the next tile overwrites the staging
                }
                continue;
            }
            float4 rs[8];  // residual of the chunk about to be stored, loaded one chunk ahead
            if constexpr (MODE == kOutF32Vec) load_residual_vec4(rs, lane, row0, n0 + 32 * half, args);
            if (!mbar_wait_bounded(smem_u32(tfull + buf), acc_phase)) {
                if (lane == 0) record_timeout(args.status, 0x400u + buf);
                break;
            }
            tc_fence_after_sync();
            int nvalid = 0;  // chunks of this warp that start inside N (uniform across the warp)
#pragma unroll
            for (int j = 0; j < kChunks; ++j)
                if (n0 + 32 * (half + 2 * j) < args.N) nvalid = j + 1;

            if constexpr (MODE == kOutF32Vec || MODE == kOutF32) {
                constexpr bool VEC4 = MODE == kOutF32Vec;
                // tcgen05.ld writes its destination registers asynchronously, until tcgen05.wait::ld: between the two the
                // compiler must not copy or recycle them, which it believes defined at the issuing statement.  Hence
                // two register sets that alternate in a loop with a compile-time trip count: a run-time loop carrying
                // ONE set over its back edge invites register moves before the wait (and the moved-from registers,
                // then free, may be handed to an address that the late write clobbers: an illegal memory access that
                // came and went with unrelated changes of this file).
                if constexpr (VEC4) {
                    // (128-bit mode: one register set in a run-time loop, as measured and tuned -- two sets spill at this
                    // kernel's 168 registers; the same exposure in principle, not observed there)
                    uint32_t r[32];
                    if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, r);
                    for (int j = 0; j < nvalid; ++j) {
                        tmem_ld_wait();
                        stage_chunk<VEC4>(r, stg, lane);
                        __syncwarp();
                        if (j + 1 < nvalid) {
                            tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), r);  // in flight during the stores below
                        } else {
                            tc_fence_before_sync();  // last chunk is out of TMEM: hand the buffer back early
                            if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                        }
                        float4 rs_cur[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) rs_cur[i] = rs[i];
                        if (j + 1 < nvalid) load_residual_vec4(rs, lane, row0, n0 + 32 * (half + 2 * (j + 1)), args);
                        store_chunk_f32<VEC4>(stg, lane, row0, n0 + 32 * (half + 2 * j), args, alpha, amax, rs_cur);
                        __syncwarp();
                    }
                } else {
                uint32_t ra[32], rb[32];
                if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, ra);
#pragma unroll
                for (int j = 0; j < kChunks; ++j) {
                    if (j < nvalid) {
                        tmem_ld_wait();
                        if (j & 1) stage_chunk<VEC4>(rb, stg, lane);
                        else stage_chunk<VEC4>(ra, stg, lane);
                        __syncwarp();
                        if (j + 1 < nvalid) {  // in flight during the stores below
                            if (j & 1) tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), ra);
                            else tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), rb);
                        } else {
                            tc_fence_before_sync();  // last chunk is out of TMEM: hand the buffer back early
                            if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                        }
                        float4 rs_cur[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) rs_cur[i] = rs[i];
                        if constexpr (VEC4)
                            if (j + 1 < nvalid) load_residual_vec4(rs, lane, row0, n0 + 32 * (half + 2 * (j + 1)), args);
                        store_chunk_f32<VEC4>(stg, lane, row0, n0 + 32 * (half + 2 * j), args, alpha, amax, rs_cur);
                        __syncwarp();
                    }
                }
                }  // !VEC4
                if (nvalid == 0) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
                }
            }
        }
        if ((args.flags & 4) && !fused) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
        }
        if constexpr (MODE == kOutF32Tma) {
            if (lane == 0) tma_store_wait_all();  // this thread's stores are complete before the CTA goes away
        }
        (void)box_it;
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---- CTA-pair variant: 256 x 256 output tile per pair of CTAs (tcgen05 cta_group::2) ---------------
//
// A 128 x 256 tile per CTA needs (128+256) x 128 operand bytes per 128-deep K block, i.e. 171 flop per byte
// pulled from L2 into shared memory; at the B200's fp8 rate that is more than the L2 can deliver, and the
// single-CTA kernel above tops out there.  Two CTAs of a cluster working on one 256 x 256 tile each load
// their own 128 rows of A and their own 128 rows (N) of W — 256 flop per byte — and the pair's leader issues
// one MMA (M = 256) that reads both CTAs' shared memory; each CTA's TMEM receives its own 128 rows, and each
// CTA runs its own epilogue.  Loads stay plain per-CTA TMA loads; only barrier arrivals cross between CTAs.
//
// BN = 256, or 192 in the fp32 modes: with N = 768 (the residual projections of a 768-wide model) 256-column
// tiles give 1.3 tiles per pair, i.e. two rounds of which the second is nearly empty; 192-column tiles give 1.73
// tiles per pair in two shorter rounds with a shorter epilogue at the end.
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(gemm_threads(MODE), 1)
gemm_fp8_tn_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_w,
                        const __grid_constant__ CUtensorMap tma_out, const GemmArgs args) {
    static_assert(BN == 256 || (BN == 192 && (MODE == kOutF32Vec || MODE == kOutF32)),
                  "192-column pair tiles exist for the st.global fp32 modes only");
    constexpr int kABytes = BM * BK, kBBytes = (BN / 2) * BK, kStageBytes = kABytes + kBBytes;
    constexpr int EW = epi_warps(MODE);
    // fp32 modes: a transpose buffer per warp; fp8 codes: bias slice + codes tile per warp; max|out| only: bias slices
    constexpr int kStagingBytes = pair_staging_bytes(MODE);
    constexpr int kTmemCols = 512;  // two accumulator buffers of BN columns; allocations are powers of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* staging = reinterpret_cast<float*>(smem + STAGES * kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes + kStagingBytes);
    uint64_t* full = bars;                // used in the leader only: both CTAs' loads report here
    uint64_t* empty = bars + STAGES;      // one set per CTA, signalled by the leader's MMA commits
    uint64_t* tfull = bars + 2 * STAGES;  // one set per CTA
    uint64_t* tempty = tfull + 2;         // used in the leader only: both CTAs' epilogue warps arrive here
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    griddep_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(tfull + b), 1);
            mbar_init(smem_u32(tempty + b), 2 * EW);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();  // the partner's barriers exist before anything arrives on them
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    griddep_wait();

    const int pair = blockIdx.x >> 1;
    const int npairs = gridDim.x >> 1;
    const int num_m = (args.M + 2 * BM - 1) / (2 * BM);
    const int num_n = (args.N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_kb = (args.K + BK - 1) / BK;

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tma_a);
            prefetch_tensormap(&tma_w);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            if constexpr (MODE == kOutF32Tma) prefetch_tensormap(&tma_out);
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                const int m0 = (tile % num_m) * 2 * BM + int(rank) * BM;
                const int n0 = (tile / num_m) * BN + int(rank) * (BN / 2);
                int ax = 0, aslab = 0;  // A's K coordinate: column inside its slab, slab index
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(empty + stage), phase ^ 1)) {
                        record_timeout(args.status, 0x2100u + (rank << 4) + stage);
                        ok = false;
                        break;
                    }
                    const uint32_t fb = map_to_cta(smem_u32(full + stage), 0);
                    uint8_t* sa = smem + stage * kStageBytes;
                    if (leader) mbar_arrive_expect_tx(smem_u32(full + stage), 2 * kStageBytes);
                    tma_load_3d_pair(smem_u32(sa), &tma_a, fb, ax, m0, aslab);
                    tma_load_2d_pair(smem_u32(sa + kABytes), &tma_w, fb, kb * BK, n0);
                    ax += BK;
                    if (ax >= args.a_slab_cols) {
                        ax = 0;
                        ++aslab;
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint64_t desc0 = make_desc_kmajor_sw128(smem_u32(smem));
            const uint32_t dhi = desc_hi(desc0), dlo0 = desc_lo(desc0);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++acc_it) {
                const uint32_t buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                if (!mbar_wait_bounded(smem_u32(tempty + buf), acc_phase ^ 1)) {
                    record_timeout(args.status, 0x2200u + buf);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(full + stage), phase)) {
                        record_timeout(args.status, 0x2300u + stage);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t alo = dlo0 + uint32_t(stage) * (kStageBytes >> 4), blo = alo + (kABytes >> 4);
                    if (kb == 0) tc_mma_f8_pair(d_tmem, desc_join(alo, dhi), desc_join(blo, dhi), args.idesc, 0);
                    else tc_mma_f8_pair_acc(d_tmem, desc_join(alo, dhi), desc_join(blo, dhi), args.idesc);
#pragma unroll
                    for (int k = 1; k < BK / 32; ++k)
                        tc_mma_f8_pair_acc(d_tmem, desc_join(alo + 2 * k, dhi), desc_join(blo + 2 * k, dhi), args.idesc);
                    // the stage is free in both CTAs once these MMAs have read it
                    tc_commit_pair(smem_u32(empty + stage));
                    tc_commit_pair(map_to_cta(smem_u32(empty + stage), 1));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) {
                    tc_commit_pair(smem_u32(tfull + buf));
                    tc_commit_pair(map_to_cta(smem_u32(tfull + buf), 1));
                }
            }
        }
    } else {
        const int e = warp - 2;
        const int q = warp & 3;
        const int half = e >> 2;
        constexpr int kChunks = BN / 64;
        float* stg = staging + e * kStagingFloatsPerWarp;
        const float alpha = ld_l2_f32(args.scale_a + 1) * ld_l2_f32(args.scale_w + 1);
        float out_q = 1.f;
        if constexpr (MODE == kOutE4M3 || MODE == kOutE5M2) {
            const float2 sc = scales_from_amax(ld_l2_f32(args.q_amax), fp8_max(MODE == kOutE4M3 ? DF8_E4M3 : DF8_E5M2));
            out_q = sc.x;
            if (blockIdx.x == 0 && e == 0 && lane == 0 && args.out_scale) {
                args.out_scale[0] = sc.x;
                args.out_scale[1] = sc.y;
            }
        }
        const uint32_t lane_addr = uint32_t(q * 32) << 16;
        auto release = [&](uint32_t buf) {  // this warp is done with accumulator buffer `buf`
            if (lane == 0) {
                if (leader) mbar_arrive(smem_u32(tempty + buf));
                else mbar_arrive_cluster(map_to_cta(smem_u32(tempty + buf), 0));
            }
        };
        uint32_t acc_it = 0;
        uint32_t box_it = 0;
        float amax = 0.f;
        for (int tile = pair; tile < num_tiles; tile += npairs, ++acc_it) {
            const uint32_t buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            const int m0 = (tile % num_m) * 2 * BM + int(rank) * BM;
            const int n0 = (tile / num_m) * BN;
            const int row0 = m0 + q * 32;
            const uint32_t taddr = tmem_base + buf * BN + lane_addr;
            if constexpr (MODE == kOutF32T) {
                auto release_buf = [&] { release(buf); };
                if (!epilogue_tile_f32_transposed<BN>(args, smem_u32(tfull + buf), acc_phase, taddr, row0, n0, half, lane,
                                                      alpha, amax, release_buf)) {
                    if (lane == 0) record_timeout(args.status, 0x2400u + (rank << 4) + buf);
                    break;
                }
                continue;
            }
            if constexpr (MODE == kOutF32Tma) {  // as in the single-CTA kernel
                uint8_t* group_boxes = reinterpret_cast<uint8_t*>(staging) + half * (8 * kTmaBoxBytes);
                float* sbias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(staging) + kEpiWarps * 2 * kTmaBoxBytes) +
                               e * kTmaBiasFloatsPerWarp;
                auto release_buf = [&] { release(buf); };
                const bool ok = epilogue_tile_f32_tma_group<BN>(&tma_out, args, group_boxes, sbias, smem_u32(tfull + buf), acc_phase,
                                                                taddr, m0, q, n0, half, lane, alpha, amax, box_it, release_buf);
                if (!ok) {
                    if (lane == 0) record_timeout(args.status, 0x2400u + (rank << 4) + buf);
                    break;
                }
                continue;
            }
            if constexpr (is_direct(MODE)) {  // as in the single-CTA kernel
                constexpr int KIND = MODE == kOutE4M3 ? int(DF8_E4M3) : (MODE == kOutE5M2 ? int(DF8_E5M2) : -1);
                constexpr int kParts = EW / 4;
                constexpr int kCh = BN / (32 * kParts);
                const int part = e >> 2;
                // this warp's columns: kCh adjacent chunks, so that its codes of a row are one contiguous segment
                const int colw = n0 + 32 * kCh * part;
                uint8_t* wst = reinterpret_cast<uint8_t*>(staging) + e * direct_staging_bytes(MODE);
                float* sb = reinterpret_cast<float*>(wst);
                uint8_t* codes_tile = wst + 256;
#pragma unroll
                for (int j = 0; j < kCh; ++j) {
                    const int col = colw + 32 * j + lane;
                    sb[j * 32 + lane] = (args.bias && col < args.N) ? __ldg(args.bias + col) : 0.f;
                }
                __syncwarp();
                if (!mbar_wait_bounded(smem_u32(tfull + buf), acc_phase)) {
                    if (lane == 0) record_timeout(args.status, 0x2400u + (rank << 4) + buf);
                    break;
                }
                tc_fence_after_sync();
                uint32_t r[kCh][32];
#pragma unroll
                for (int j = 0; j < kCh; ++j)
                    if (colw + 32 * j < args.N) tmem_ld_32x32(taddr + 32 * (kCh * part + j), r[j]);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                release(buf);
                const int grow = row0 + lane;
#pragma unroll
                for (int j = 0; j < kCh; ++j) {
                    const int col0 = colw + 32 * j;
                    if (col0 < args.N)
                        direct_chunk<KIND, 2 * kCh>(r[j], grow, col0, args, alpha, out_q, amax, sb + j * 32, codes_tile, j);
                }
                __syncwarp();
                if constexpr (KIND >= 0) {
                    store_staged_codes<2 * kCh>(codes_tile, lane, row0, colw, args);
                    __syncwarp();
                }
                continue;
            }
            float4 rs[8];
            if constexpr (MODE == kOutF32Vec) load_residual_vec4(rs, lane, row0, n0 + 32 * half, args);
            if (!mbar_wait_bounded(smem_u32(tfull + buf), acc_phase)) {
                if (lane == 0) record_timeout(args.status, 0x2400u + (rank << 4) + buf);
                break;
            }
            tc_fence_after_sync();
            int nvalid = 0;
#pragma unroll
            for (int j = 0; j < kChunks; ++j)
                if (n0 + 32 * (half + 2 * j) < args.N) nvalid = j + 1;

            if constexpr (MODE == kOutF32Vec || MODE == kOutF32) {
                constexpr bool VEC4 = MODE == kOutF32Vec;
                if constexpr (VEC4) {
                    // (one register set in a run-time loop: see the single-CTA kernel)
                    uint32_t r[32];
                    if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, r);
                    for (int j = 0; j < nvalid; ++j) {
                        tmem_ld_wait();
                        stage_chunk<VEC4>(r, stg, lane);
                        __syncwarp();
                        if (j + 1 < nvalid) {
                            tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), r);
                        } else {
                            tc_fence_before_sync();
                            release(buf);
                        }
                        float4 rs_cur[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) rs_cur[i] = rs[i];
                        if (j + 1 < nvalid) load_residual_vec4(rs, lane, row0, n0 + 32 * (half + 2 * (j + 1)), args);
                        store_chunk_f32<VEC4>(stg, lane, row0, n0 + 32 * (half + 2 * j), args, alpha, amax, rs_cur);
                        __syncwarp();
                    }
                } else {
                // (two register sets and a compile-time trip count: see the single-CTA kernel)
                uint32_t ra[32], rb[32];
                if (nvalid > 0) tmem_ld_32x32(taddr + 32 * half, ra);
#pragma unroll
                for (int j = 0; j < kChunks; ++j) {
                    if (j < nvalid) {
                        tmem_ld_wait();
                        if (j & 1) stage_chunk<VEC4>(rb, stg, lane);
                        else stage_chunk<VEC4>(ra, stg, lane);
                        __syncwarp();
                        if (j + 1 < nvalid) {
                            if (j & 1) tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), ra);
                            else tmem_ld_32x32(taddr + 32 * (half + 2 * (j + 1)), rb);
                        } else {
                            tc_fence_before_sync();
                            release(buf);
                        }
                        float4 rs_cur[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) rs_cur[i] = rs[i];
                        if constexpr (VEC4)
                            if (j + 1 < nvalid) load_residual_vec4(rs, lane, row0, n0 + 32 * (half + 2 * (j + 1)), args);
                        store_chunk_f32<VEC4>(stg, lane, row0, n0 + 32 * (half + 2 * j), args, alpha, amax, rs_cur);
                        __syncwarp();
                    }
                }
                }  // !VEC4
                if (nvalid == 0) {
                    tc_fence_before_sync();
                    __syncwarp();
                    release(buf);
                }
            }
        }
        if (args.flags & 4) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
        }
        if constexpr (MODE == kOutF32Tma) {
            if (lane == 0) tma_store_wait_all();
        }
        (void)box_it;
    }

    // neither CTA may leave while its partner can still read its shared memory or signal its barriers
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <int BN, int MODE>
struct PairCfg {
    // ring depth: the operand loads are latency-bound (~2.4 k cycles from issue to arrival with every SM loading),
    // so as many stages as fit beside the epilogue's staging
    static constexpr int kStages = MODE == kOutF32Tma ? 4 : ((BN == 192 || MODE == kOutNone || MODE == kOutF32T) ? 6 : 5);
    static constexpr int kSmemBytes = kStages * (BM * BK + (BN / 2) * BK) + pair_staging_bytes(MODE) + 256 + 1024;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

template <int BN, int MODE>
df8_status launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const GemmArgs& args,
                            int grid, cudaStream_t st) {
    constexpr int kPairSmemBytes = PairCfg<BN, MODE>::kSmemBytes;
    auto kern = gemm_fp8_tn_pair_kernel<BN, PairCfg<BN, MODE>::kStages, MODE>;
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        DF8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid), 1, 1);
    cfg.blockDim = dim3(gemm_threads(MODE), 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, ta, tw, to, args);
    if (err != cudaSuccess)
        return fail(DF8_ERR_CUDA, "launch of gemm_fp8_tn_pair_kernel failed: %s", cudaGetErrorString(err));
    return DF8_OK;
}

template <int BN, int STAGES, int MODE>
df8_status launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const GemmArgs& args,
                       int grid, cudaStream_t st) {
    using Cfg = GemmCfg<BN, STAGES, MODE>;
    auto kern = gemm_fp8_tn_kernel<BN, STAGES, MODE>;
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        DF8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        if constexpr (MODE == kOutE4M3 || MODE == kOutE5M2)
            DF8_CUDA_TRY(cudaFuncSetAttribute(gemm_fp8_tn_kernel<BN, STAGES, MODE, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        configured[dev] = true;
    }
    if (args.grid_counter != nullptr) {
        if constexpr (MODE == kOutE4M3 || MODE == kOutE5M2) {
        auto fkern = gemm_fp8_tn_kernel<BN, STAGES, MODE, true>;
        // fused launch: its grid-wide barrier needs every CTA resident, i.e. a cooperative launch
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(grid));
        cfg.blockDim = dim3(gemm_threads(MODE));
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t err = cudaLaunchKernelEx(&cfg, fkern, ta, tw, to, args);
        if (err != cudaSuccess) {
            (void)cudaGetLastError();
            return DF8_ERR_UNSUPPORTED;  // not co-schedulable here: the caller falls back to two launches
        }
        return DF8_OK;
        } else {
            return fail(DF8_ERR_INVALID, "the one-launch form exists for the fp8 output modes only");
        }
    }
    cudaError_t err = launch_kernel(kern, dim3(unsigned(grid)), dim3(gemm_threads(MODE)), Cfg::kSmemBytes, st, ta, tw, to, args);
    if (err != cudaSuccess) return fail(DF8_ERR_CUDA, "launch of gemm_fp8_tn_kernel failed: %s", cudaGetErrorString(err));
    return DF8_OK;
}

template <int MODE>
df8_status launch_gemm_bn(bool wide, const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to,
                          const GemmArgs& args, int grid, cudaStream_t st) {
    // ring depth: whatever fits beside the epilogue's staging.  One K block of operands takes ~1300 cycles to
    // arrive from L2 and ~512 (256 at BN = 128) to consume, so three 48 KB stages leave the tensor core waiting;
    // the fp8 / amax modes need no transpose buffer and get a deeper ring.
    if constexpr (MODE == kOutNone)
        return wide ? launch_gemm<256, 4, MODE>(ta, tw, to, args, grid, st) : launch_gemm<128, 6, MODE>(ta, tw, to, args, grid, st);
    else if constexpr (MODE == kOutF32Tma)  // 256-column tiles only (run_gemm falls back to the st.global modes otherwise)
        return launch_gemm<256, 3, MODE>(ta, tw, to, args, grid, st);
    else if constexpr (MODE == kOutF32T)  // no staging: the whole of shared memory is operand ring
        return wide ? launch_gemm<256, 4, MODE>(ta, tw, to, args, grid, st) : launch_gemm<128, 6, MODE>(ta, tw, to, args, grid, st);
    else
        return wide ? launch_gemm<256, 3, MODE>(ta, tw, to, args, grid, st) : launch_gemm<128, 5, MODE>(ta, tw, to, args, grid, st);
}

// DF8_GEMM_PAIR=0 / 1 in the environment (read at every call) forces the choice for profiling and tests;
// otherwise the pair kernel takes problems that give every CTA pair at least one full 256 x 256 tile.
bool use_pair_kernel(int M, int N, int K, int sms, int mode) {
    const char* e = getenv("DF8_GEMM_PAIR");
    if (e && e[0] == '0') return false;
    if (e && e[0] == '1') return M > 0 && N > 0;
    // Outputs far larger than L2 written through TMA stores (the vocabulary head: 1.6 GB of logits): the tile's
    // stores are the longest phase and slow the operand loads of the next tile down; a pair loads half of W per
    // CTA and hides more of them.  Measured at 8192 x 50257 x 768 into rows of 50272 floats: 462 us with pairs,
    // 598 us without (and 578 us for dense rows of 50257 floats through 4-byte stores); at 8192 x 2304 x 768 the
    // single-CTA kernel stays ahead (30 against 33 us).
    if ((mode == kOutF32Tma || mode == kOutF32T) && M >= 256 && N >= 256 && double(M) * double(N) * 4.0 >= 512e6) return true;
    // measured on B200 (M = 8192): 8192 x 8192 x 8192 runs at 2547 TFLOP/s with CTA pairs against 2245 without;
    // at K = 768 the epilogue dominates and the pairs' coupled accumulator hand-back costs a few per cent
    // the max|out| / codes passes at K = 1024 stay ahead on single CTAs (8192 x 3072 x 1024, both passes: 51.5 against
    // 55.3 us; 8192 x 4096 x 1024: 67.0 against 69.8), the fp32 outputs at K = 3072 on pairs (27.1 against 31.2 us)
    const long tiles2 = long((M + 255) / 256) * ((N + 255) / 256);
    const int k_min = is_direct(mode) ? 2048 : 1024;
    return K >= k_min && M >= 256 && N >= 256 && tiles2 >= sms / 2;
}

// Shared host path of the entry points: picks the tile width, encodes the tensor maps, launches `mode`.
// `a_slabs`: A's K dimension is stored as that many row-major [M, K / a_slabs] slabs, M * K / a_slabs bytes apart
// (what an all-gather of per-rank column slices leaves); 1 = an ordinary [M, K] matrix.
// `tma_fallback`: the st.global fp32 mode to use where the TMA-store mode does not apply (narrow tiles).
// `fused`: in: try the one-launch max|out| + codes form (fp8 modes); out: whether that is what was launched.  When
// it cannot be (CTA-pair shapes, fewer tiles than SMs, no cooperative launch) nothing is launched and the caller
// runs the two passes.
df8_status run_gemm(int mode, const uint8_t* a_codes, df8_kind kind_a, const uint8_t* w_codes, df8_kind kind_w,
                    GemmArgs args, cudaStream_t st, bool* fused = nullptr, int a_slabs = 1,
                    int tma_fallback = kOutF32, int a_slab_rows = 0) {
    const int M = args.M, N = args.N, K = args.K;
    df8_status src = status_word_device_ptr(&args.status);
    if (src != DF8_OK) return src;
    const bool want_fused = fused != nullptr && *fused;
    if (fused) *fused = false;
    if (a_slabs < 1 || K % a_slabs != 0 || (a_slabs > 1 && (K / a_slabs) % BK != 0))
        return fail(DF8_ERR_UNSUPPORTED, "fp8 GEMM: K=%d cannot be read as %d slabs (a slab must be a multiple of %d columns)",
                    K, a_slabs, BK);
    const int slab_cols = K / a_slabs;
    args.a_slab_cols = slab_cols;
    if (args.ldc == 0) args.ldc = N;
    if (const char* e = getenv("DF8_GEMM_TMA_STORE"))  // profiling and tests: 0 keeps the st.global epilogues
        if (e[0] == '0' && mode == kOutF32Tma) mode = tma_fallback;

    const int sms = sm_count();
    // A: coordinates (column inside the slab, row, slab)
    CUtensorMap ta, tw, to = {};
    // a_slab_rows: the slabs hold that many rows each (M of them are used): a row range of a gathered tensor
    if (a_slab_rows != 0 && a_slab_rows < M)
        return fail(DF8_ERR_INVALID, "fp8 GEMM: a_slab_rows=%d is smaller than M=%d", a_slab_rows, M);
    const uint64_t slab_rows = a_slab_rows ? uint64_t(a_slab_rows) : uint64_t(M);
    df8_status rc = make_tmap_3d_u8(&ta, a_codes, uint64_t(M), uint64_t(slab_cols), uint64_t(a_slabs), uint64_t(slab_cols),
                                    slab_rows * uint64_t(slab_cols), BM, BK, 128);
    if (rc != DF8_OK) return rc;
    auto make_out_map = [&]() {
        return make_tmap_2d_f32(&to, args.out, uint64_t(M), uint64_t(N), uint64_t(args.ldc) * sizeof(float), 128, 32, 128);
    };
    // CTA pairs on 256 x 256 tiles when the problem fills them (see gemm_fp8_tn_pair_kernel)
    if (use_pair_kernel(M, N, K, sms, mode)) {
        if (want_fused) return DF8_OK;
        // Tile width of the fp32 modes, by the measured per-K-block and per-chunk costs (cycles): a K block is
        // bound by the tensor core (2 BN) or by the CTA's operand bytes arriving at ~50 bytes per cycle while the
        // previous tile's stores are in flight; a 32-column chunk of the epilogue takes a warp ~2500 cycles and
        // the last tile's epilogue overlaps nothing.
        auto pair_cost = [&](int bn) {
            const long tiles = long((M + 255) / 256) * ((N + bn - 1) / bn);
            const double rounds = double((tiles + sms / 2 - 1) / (sms / 2));
            const double mma = 2.0 * bn, loads = (BM * BK + bn / 2 * BK) / 50.0;
            return rounds * double((K + BK - 1) / BK) * (mma > loads ? mma : loads) + 2500.0 * (bn / 64);
        };
        const bool fp32_mode = mode == kOutF32Vec || mode == kOutF32;
        int bn2 = fp32_mode && pair_cost(192) < pair_cost(256) ? 192 : 256;
        if (const char* e = getenv("DF8_GEMM_PAIR_BN")) {  // profiling and tests
            if (fp32_mode && atoi(e) == 192) bn2 = 192;
            if (atoi(e) == 256) bn2 = 256;
        }
        const long tiles2 = long((M + 255) / 256) * ((N + bn2 - 1) / bn2);
        const long pairs = tiles2 < sms / 2 ? tiles2 : sms / 2;
        rc = make_tmap_2d_u8(&tw, w_codes, uint64_t(N), uint64_t(K), uint64_t(K), uint32_t(bn2 / 2), BK, 128);
        if (rc != DF8_OK) return rc;
        if (mode == kOutF32Tma && (rc = make_out_map()) != DF8_OK) return rc;
        args.idesc = ptx::make_idesc_f8(256, bn2, int(kind_a), int(kind_w));
        const int grid2 = int(pairs) * 2;
        switch (mode) {
            case kOutF32Vec:
                return bn2 == 192 ? launch_gemm_pair<192, kOutF32Vec>(ta, tw, to, args, grid2, st)
                                  : launch_gemm_pair<256, kOutF32Vec>(ta, tw, to, args, grid2, st);
            case kOutF32:
                return bn2 == 192 ? launch_gemm_pair<192, kOutF32>(ta, tw, to, args, grid2, st)
                                  : launch_gemm_pair<256, kOutF32>(ta, tw, to, args, grid2, st);
            case kOutF32Tma: return launch_gemm_pair<256, kOutF32Tma>(ta, tw, to, args, grid2, st);
            case kOutF32T: return launch_gemm_pair<256, kOutF32T>(ta, tw, to, args, grid2, st);
            case kOutE4M3: return launch_gemm_pair<256, kOutE4M3>(ta, tw, to, args, grid2, st);
            case kOutE5M2: return launch_gemm_pair<256, kOutE5M2>(ta, tw, to, args, grid2, st);
            default: return launch_gemm_pair<256, kOutNone>(ta, tw, to, args, grid2, st);
        }
    }
    // Tile width.  A TMA tiled load costs the SM's copy engine ~250 cycles whatever its size, and L2 delivers
    // ~85 bytes per cycle to an SM: a 128 x 128 K block (two loads, 32 KB) therefore takes ~530 cycles although
    // its MMAs need 256, about as long as a 128 x 256 one (48 KB, MMAs 512).  So narrow tiles only pay when
    // they save whole rounds of the persistent grid.
    // The st.global fp32 modes add their epilogue to the picture: a 32 x 32 chunk takes a warp ~2000 cycles to
    // stage and store (measured), i.e. ~31 cycles per tile column with eight warps, which exceeds the main loop at
    // small K.
    auto rounds = [&](int bn) {
        const long tiles = long((M + BM - 1) / BM) * ((N + bn - 1) / bn);
        return double((tiles + sms - 1) / sms);
    };
    const double kloop = double((K + BK - 1) / BK) * 540.0;
    const int cost_mode = mode == kOutF32Tma ? tma_fallback : mode;
    auto tile_cycles = [&](int bn) {
        const double main_loop = bn == 256 ? kloop : 0.94 * kloop;
        const double epilogue = (cost_mode == kOutF32Vec || cost_mode == kOutF32) ? 31.0 * bn : 0.0;
        return main_loop > epilogue ? main_loop : epilogue;
    };
    const bool wide = N > 128 && rounds(256) * tile_cycles(256) <= rounds(128) * tile_cycles(128);
    if (mode == kOutF32Tma && !wide) mode = tma_fallback;  // the TMA-store epilogue exists for 256-column tiles
    const int bn = wide ? 256 : 128;
    const long tiles = long((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int grid = int(tiles < sms ? tiles : sms);

    rc = make_tmap_2d_u8(&tw, w_codes, uint64_t(N), uint64_t(K), uint64_t(K), uint32_t(bn), BK, 128);
    if (rc != DF8_OK) return rc;
    if (mode == kOutF32Tma && (rc = make_out_map()) != DF8_OK) return rc;
    args.idesc = ptx::make_idesc_f8(BM, bn, int(kind_a), int(kind_w));
    if (want_fused) {
        if (grid != sms || (mode != kOutE4M3 && mode != kOutE5M2)) return DF8_OK;  // nothing launched, *fused stays false
        static std::atomic<unsigned int> next_slot{0};
        unsigned int* counters = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&counters), g_gemm_grid_counter) != cudaSuccess) {
            (void)cudaGetLastError();
            return DF8_OK;
        }
        args.grid_counter = counters + next_slot.fetch_add(1u) % unsigned(kFusedCounters);
        const df8_status rcf = mode == kOutE4M3 ? launch_gemm_bn<kOutE4M3>(wide, ta, tw, to, args, grid, st)
                                                : launch_gemm_bn<kOutE5M2>(wide, ta, tw, to, args, grid, st);
        if (rcf == DF8_ERR_UNSUPPORTED) return DF8_OK;  // no cooperative launch here: two passes
        if (rcf == DF8_OK) *fused = true;
        return rcf;
    }

    switch (mode) {
        case kOutF32Vec: return launch_gemm_bn<kOutF32Vec>(wide, ta, tw, to, args, grid, st);
        case kOutF32: return launch_gemm_bn<kOutF32>(wide, ta, tw, to, args, grid, st);
        case kOutF32Tma: return launch_gemm_bn<kOutF32Tma>(wide, ta, tw, to, args, grid, st);
        case kOutF32T: return launch_gemm_bn<kOutF32T>(wide, ta, tw, to, args, grid, st);
        case kOutE4M3: return launch_gemm_bn<kOutE4M3>(wide, ta, tw, to, args, grid, st);
        case kOutE5M2: return launch_gemm_bn<kOutE5M2>(wide, ta, tw, to, args, grid, st);
        default: return launch_gemm_bn<kOutNone>(wide, ta, tw, to, args, grid, st);
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_gemm_fp8_tn(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                      const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                      const float* bias, const float* residual, int M, int N, int K, int flags,
                                      float* out, float* out_amax, df8_stream stream) {
    return df8_gemm_fp8_tn_ex(a_codes, kind_a, scale_a, 1, w_codes, kind_w, scale_w, bias, residual, M, N, K, flags, out,
                              N, out_amax, stream);
}

extern "C" df8_status df8_gemm_fp8_tn_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                         const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                         const float* bias, const float* residual, int M, int N, int K, int flags,
                                         float* out, int ldc, float* out_amax, df8_stream stream) {
    return df8_gemm_fp8_tn_part(a_codes, kind_a, scale_a, a_slabs, M, w_codes, kind_w, scale_w, bias, residual, M, N, K, flags,
                                out, ldc, out_amax, stream);
}

extern "C" df8_status df8_gemm_fp8_tn_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                           int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                           const float* bias, const float* residual, int M, int N, int K, int flags,
                                           float* out, int ldc, float* out_amax, df8_stream stream) {
    DF8_REQUIRE((kind_a == DF8_E4M3 || kind_a == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2),
                "df8_gemm_fp8_tn: unknown fp8 kind");
    DF8_REQUIRE(ldc >= N, "df8_gemm_fp8_tn: ldc=%d is smaller than N=%d", ldc, N);
    DF8_REQUIRE(M >= 0 && N >= 0 && K > 0, "df8_gemm_fp8_tn: bad shape M=%d N=%d K=%d", M, N, K);
    DF8_REQUIRE((flags & ~7) == 0, "df8_gemm_fp8_tn: unknown flags 0x%x", flags);
    cudaStream_t st = as_stream(stream);
    if (flags & DF8_EPI_AMAX) {
        DF8_REQUIRE(out_amax != nullptr, "df8_gemm_fp8_tn: DF8_EPI_AMAX needs out_amax");
        DF8_CLEAR_AMAX(out_amax, st);
    }
    if (M == 0 || N == 0) return DF8_OK;
    DF8_REQUIRE(a_codes && w_codes && scale_a && scale_w && out, "df8_gemm_fp8_tn: null buffer");
    DF8_REQUIRE(!(flags & DF8_EPI_RESIDUAL) || residual != nullptr, "df8_gemm_fp8_tn: DF8_EPI_RESIDUAL needs residual");
    if (K % 16 != 0)
        return fail(DF8_ERR_UNSUPPORTED, "df8_gemm_fp8_tn: K=%d must be a multiple of 16 (TMA row pitch)", K);

    GemmArgs args{};
    args.scale_a = scale_a;
    args.scale_w = scale_w;
    args.bias = bias;
    args.residual = residual;
    args.out = out;
    args.out_amax = out_amax;
    args.M = M;
    args.N = N;
    args.K = K;
    args.ldc = ldc;
    args.flags = flags;
    // 128-bit accesses need rows that start on 16-byte boundaries (a pitch that is a multiple of 4 floats; N itself
    // may be anything: the last group of a row then reaches into the pitch padding)
    const bool pitch4 = ldc % 4 == 0 && ldc >= (N + 3) / 4 * 4;
    const bool vec4 = pitch4 && aligned16(out) && (!bias || aligned16(bias)) &&
                      (!(flags & DF8_EPI_RESIDUAL) || aligned16(residual));
    const int st_mode = vec4 ? kOutF32Vec : kOutF32;
    // without a residual to read, rows that start on 16-byte boundaries leave through TMA stores
    const bool tma = pitch4 && aligned16(out) && !(flags & DF8_EPI_RESIDUAL);
    // Operands swapped (the kernel's A = the weight matrix, accumulator tile = [128 features, tokens], see kOutF32T):
    // a lane then owns one output COLUMN and a warp's store instruction covers 128 contiguous bytes of one output row
    // straight from registers, with no staging in shared memory and no alignment rule for N or ldc; results are bit
    // for bit those of the other epilogues (tested).  Measured at M = 8192, each shape alone (us, plain -> swapped):
    // fp32 output with GELU 8192 x 3072 x 768: 68 -> 40; out-projection 768 x 768 with residual 17.6 -> 15.7; FC2
    // 768 x 3072: 35.8 -> 35.0; 8192 x 8192 x 8192: 450 -> 413; QKV-shaped 2304 x 768: the same; the vocabulary head
    // into pitched rows (TMA stores) 394 -> 417, into dense rows of 50257 floats 565 -> 615.  Inside the GPT-2 small
    // forward, though, the swapped out-projection and FC2 made the pass SLOWER (3.435 against 3.346 ms, two runs
    // each), so only the case with the large margin takes this path by itself: GELU outputs.
    // DF8_GEMM_SWAP=0 / 1 in the environment forces the choice, 2 = every output that is not far larger than L2
    // (profiling and tests).
    {
        const char* e = getenv("DF8_GEMM_SWAP");
        bool swap = a_slabs == 1 && (flags & DF8_EPI_GELU) && M >= 256 && N >= 256 && double(M) * double(N) * 4.0 < 512e6;
        if (e && e[0] == '0') swap = false;
        if (e && e[0] == '1') swap = a_slabs == 1;
        if (e && e[0] == '2') swap = a_slabs == 1 && M >= 256 && N >= 256 && double(M) * double(N) * 4.0 < 512e6;
        if (swap) {
            args.scale_a = scale_w;
            args.scale_w = scale_a;
            args.M = N;
            args.N = M;
            return run_gemm(kOutF32T, w_codes, kind_w, a_codes, kind_a, args, st);
        }
    }
    return run_gemm(tma ? kOutF32Tma : st_mode, a_codes, kind_a, w_codes, kind_w, args, st, nullptr, a_slabs, st_mode,
                    a_slab_rows);
}

extern "C" df8_status df8_gemm_fp8_tn_q(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                        const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                        const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                                        uint8_t* out_codes, float* out_scale, float* out_amax, df8_stream stream) {
    DF8_REQUIRE((kind_a == DF8_E4M3 || kind_a == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2) &&
                    (out_kind == DF8_E4M3 || out_kind == DF8_E5M2),
                "df8_gemm_fp8_tn_q: unknown fp8 kind");
    DF8_REQUIRE(M >= 0 && N >= 0 && K > 0, "df8_gemm_fp8_tn_q: bad shape M=%d N=%d K=%d", M, N, K);
    DF8_REQUIRE((flags & ~DF8_EPI_GELU) == 0, "df8_gemm_fp8_tn_q: only DF8_EPI_GELU is accepted, got 0x%x", flags);
    DF8_REQUIRE(out_amax && out_scale, "df8_gemm_fp8_tn_q: out_amax and out_scale are required");
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(out_amax, st);
    if (K % 16 != 0 || N % 32 != 0)
        return fail(DF8_ERR_UNSUPPORTED, "df8_gemm_fp8_tn_q: needs K %% 16 == 0 and N %% 32 == 0 (K=%d N=%d)", K, N);
    DF8_REQUIRE(M == 0 || N == 0 || (a_codes && w_codes && scale_a && scale_w && out_codes),
                "df8_gemm_fp8_tn_q: null buffer");
    DF8_REQUIRE(aligned16(out_codes) && (!bias || aligned16(bias)), "df8_gemm_fp8_tn_q: out_codes and bias must be 16-byte aligned");

    GemmArgs args{};
    args.scale_a = scale_a;
    args.scale_w = scale_w;
    args.bias = bias;
    args.out_amax = out_amax;
    args.M = M;
    args.N = N;
    args.K = K;
    args.out_codes = out_codes;
    args.q_amax = out_amax;
    args.out_scale = out_scale;
    if (M == 0 || N == 0) {  // still publish the scale of an empty tensor: {1, 1}
        const float one[2] = {1.f, 1.f};
        DF8_CUDA_TRY(cudaMemcpyAsync(out_scale, one, sizeof(one), cudaMemcpyHostToDevice, st));
        return DF8_OK;
    }
    // With DF8_GEMM_FUSED_Q=1 in the environment, one launch when the problem qualifies (single-CTA tiles, at least
    // one tile per SM): max|out| over all tiles, a grid-wide barrier, then the codes, with each CTA's last two
    // accumulator tiles kept in TMEM across the barrier instead of being computed twice.  Not the default: back to
    // back it saves 2-4 us per product (34.0 against 35.7 us at 8192 x 2304 x 768), but inside a GPT-2 small forward
    // the cooperative launches and the wait of every launch for its slowest CTA cost more than that (3.56 against
    // 3.52 ms per forward), and about one process in three ran another 0.1-0.4 ms slower for its whole life where
    // the two launches are steady to 0.1 %.
    {
        const char* e = getenv("DF8_GEMM_FUSED_Q");
        bool fused = e && e[0] == '1';
        if (fused) {
            args.flags = flags;
            df8_status rcf = run_gemm(out_kind == DF8_E4M3 ? kOutE4M3 : kOutE5M2, a_codes, kind_a, w_codes, kind_w, args, st, &fused);
            if (rcf != DF8_OK) return rcf;
            if (fused) return DF8_OK;
        }
    }
    // pass 1: max|out| only;  pass 2: the same product again, quantised with the scale that max gives
    args.flags = flags | DF8_EPI_AMAX;
    df8_status rc = run_gemm(kOutNone, a_codes, kind_a, w_codes, kind_w, args, st);
    if (rc != DF8_OK) return rc;
    args.flags = flags;
    return run_gemm(out_kind == DF8_E4M3 ? kOutE4M3 : kOutE5M2, a_codes, kind_a, w_codes, kind_w, args, st);
}

// The two halves of df8_gemm_fp8_tn_q as separate calls, for callers that have to combine the max|out|
// with other ranks' (column-sharded layers) between the passes.
extern "C" df8_status df8_gemm_fp8_tn_amax(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                           const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                           const float* bias, int M, int N, int K, int flags, float* out_amax,
                                           df8_stream stream) {
    return df8_gemm_fp8_tn_amax_ex(a_codes, kind_a, scale_a, 1, w_codes, kind_w, scale_w, bias, M, N, K, flags, out_amax,
                                   stream);
}

extern "C" df8_status df8_gemm_fp8_tn_amax_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                              const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                              const float* bias, int M, int N, int K, int flags, float* out_amax,
                                              df8_stream stream) {
    return df8_gemm_fp8_tn_amax_part(a_codes, kind_a, scale_a, a_slabs, M, w_codes, kind_w, scale_w, bias, M, N, K, flags,
                                     out_amax, stream);
}

extern "C" df8_status df8_gemm_fp8_tn_amax_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                                int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w,
                                                const float* scale_w, const float* bias, int M, int N, int K, int flags,
                                                float* out_amax, df8_stream stream) {
    DF8_REQUIRE((kind_a == DF8_E4M3 || kind_a == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2),
                "df8_gemm_fp8_tn_amax: unknown fp8 kind");
    DF8_REQUIRE(M >= 0 && N >= 0 && K > 0, "df8_gemm_fp8_tn_amax: bad shape M=%d N=%d K=%d", M, N, K);
    DF8_REQUIRE((flags & ~DF8_EPI_GELU) == 0, "df8_gemm_fp8_tn_amax: only DF8_EPI_GELU is accepted, got 0x%x", flags);
    DF8_REQUIRE(out_amax != nullptr, "df8_gemm_fp8_tn_amax: out_amax is required");
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(out_amax, st);
    if (M == 0 || N == 0) return DF8_OK;
    if (K % 16 != 0 || N % 32 != 0)
        return fail(DF8_ERR_UNSUPPORTED, "df8_gemm_fp8_tn_amax: needs K %% 16 == 0 and N %% 32 == 0 (K=%d N=%d)", K, N);
    DF8_REQUIRE(a_codes && w_codes && scale_a && scale_w, "df8_gemm_fp8_tn_amax: null buffer");
    DF8_REQUIRE(!bias || aligned16(bias), "df8_gemm_fp8_tn_amax: bias must be 16-byte aligned");
    GemmArgs args{};
    args.scale_a = scale_a;
    args.scale_w = scale_w;
    args.bias = bias;
    args.out_amax = out_amax;
    args.M = M;
    args.N = N;
    args.K = K;
    args.flags = flags | DF8_EPI_AMAX;
    return run_gemm(kOutNone, a_codes, kind_a, w_codes, kind_w, args, st, nullptr, a_slabs, kOutF32, a_slab_rows);
}

extern "C" df8_status df8_gemm_fp8_tn_codes(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                            const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                            const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                                            const float* amax_in, uint8_t* out_codes, float* out_scale,
                                            df8_stream stream) {
    return df8_gemm_fp8_tn_codes_ex(a_codes, kind_a, scale_a, 1, w_codes, kind_w, scale_w, bias, M, N, K, flags, out_kind,
                                    amax_in, out_codes, out_scale, stream);
}

extern "C" df8_status df8_gemm_fp8_tn_codes_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                               const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                               const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                                               const float* amax_in, uint8_t* out_codes, float* out_scale,
                                               df8_stream stream) {
    return df8_gemm_fp8_tn_codes_part(a_codes, kind_a, scale_a, a_slabs, M, w_codes, kind_w, scale_w, bias, M, N, K, flags,
                                      out_kind, amax_in, out_codes, out_scale, stream);
}

extern "C" df8_status df8_gemm_fp8_tn_codes_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                                 int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w,
                                                 const float* scale_w, const float* bias, int M, int N, int K, int flags,
                                                 df8_kind out_kind, const float* amax_in, uint8_t* out_codes,
                                                 float* out_scale, df8_stream stream) {
    DF8_REQUIRE((kind_a == DF8_E4M3 || kind_a == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2) &&
                    (out_kind == DF8_E4M3 || out_kind == DF8_E5M2),
                "df8_gemm_fp8_tn_codes: unknown fp8 kind");
    DF8_REQUIRE(M >= 0 && N >= 0 && K > 0, "df8_gemm_fp8_tn_codes: bad shape M=%d N=%d K=%d", M, N, K);
    DF8_REQUIRE((flags & ~DF8_EPI_GELU) == 0, "df8_gemm_fp8_tn_codes: only DF8_EPI_GELU is accepted, got 0x%x", flags);
    DF8_REQUIRE(amax_in != nullptr, "df8_gemm_fp8_tn_codes: amax_in is required");
    if (M == 0 || N == 0) return DF8_OK;
    if (K % 16 != 0 || N % 32 != 0)
        return fail(DF8_ERR_UNSUPPORTED, "df8_gemm_fp8_tn_codes: needs K %% 16 == 0 and N %% 32 == 0 (K=%d N=%d)", K, N);
    DF8_REQUIRE(a_codes && w_codes && scale_a && scale_w && out_codes, "df8_gemm_fp8_tn_codes: null buffer");
    DF8_REQUIRE(aligned16(out_codes) && (!bias || aligned16(bias)),
                "df8_gemm_fp8_tn_codes: out_codes and bias must be 16-byte aligned");
    GemmArgs args{};
    args.scale_a = scale_a;
    args.scale_w = scale_w;
    args.bias = bias;
    args.M = M;
    args.N = N;
    args.K = K;
    args.flags = flags;
    args.out_codes = out_codes;
    args.q_amax = amax_in;
    args.out_scale = out_scale;
    return run_gemm(out_kind == DF8_E4M3 ? kOutE4M3 : kOutE5M2, a_codes, kind_a, w_codes, kind_w, args, as_stream(stream),
                    nullptr, a_slabs, kOutF32, a_slab_rows);
}

// The skinny product of a decode step: out[B, N] = epi(X[B, K] . W[N, K]^T * dq + bias), B <= 128 token rows against a
// whole weight matrix.  Bound by streaming W from HBM; computed as W . X^T (the weight rows fill the 128-row
// tensor-core tile, the batch is the tile's N) and written back transposed.
extern "C" df8_status df8_gemv_fp8_tn(const uint8_t* x_codes, df8_kind kind_x, const float* scale_x,
                                      const uint8_t* w_codes, df8_kind kind_w, const float* scale_w, const float* bias,
                                      const float* residual, int B, int N, int K, int flags, float* out, float* out_amax,
                                      df8_stream stream) {
    DF8_REQUIRE((kind_x == DF8_E4M3 || kind_x == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2),
                "df8_gemv_fp8_tn: unknown fp8 kind");
    DF8_REQUIRE(B >= 0 && N >= 0 && K > 0, "df8_gemv_fp8_tn: bad shape B=%d N=%d K=%d", B, N, K);
    DF8_REQUIRE((flags & ~7) == 0, "df8_gemv_fp8_tn: unknown flags 0x%x", flags);
    cudaStream_t st = as_stream(stream);
    if (flags & DF8_EPI_AMAX) {
        DF8_REQUIRE(out_amax != nullptr, "df8_gemv_fp8_tn: DF8_EPI_AMAX needs out_amax");
        DF8_CLEAR_AMAX(out_amax, st);
    }
    if (B == 0 || N == 0) return DF8_OK;
    if (B > 128) return fail(DF8_ERR_UNSUPPORTED, "df8_gemv_fp8_tn: at most 128 token rows (got %d); use df8_gemm_fp8_tn", B);
    if (K % 16 != 0) return fail(DF8_ERR_UNSUPPORTED, "df8_gemv_fp8_tn: K=%d must be a multiple of 16 (TMA row pitch)", K);
    DF8_REQUIRE(x_codes && w_codes && scale_x && scale_w && out, "df8_gemv_fp8_tn: null buffer");
    DF8_REQUIRE(!(flags & DF8_EPI_RESIDUAL) || residual != nullptr, "df8_gemv_fp8_tn: DF8_EPI_RESIDUAL needs residual");
    GemmArgs args{};
    args.scale_a = scale_w;  // the roles are swapped: the kernel's A operand is the weight matrix
    args.scale_w = scale_x;
    args.bias = bias;
    args.residual = residual;
    args.out = out;
    args.out_amax = out_amax;
    args.M = N;
    args.N = B;
    args.K = K;
    args.ldc = N;
    args.flags = flags;
    return run_gemm(kOutF32T, w_codes, kind_w, x_codes, kind_x, args, st);
}

