// fp8 multi-head attention for sm_100a: QK^T, online softmax and PV in one kernel, on tcgen05.
//
// Input is the fused QKV projection output as fp8 codes, [B*T, 3E] row-major with Q = columns [0,E),
// K = [E,2E), V = [2E,3E) and head h = columns [hD,(h+1)D) of each — the layout upstream's
// MultiHeadAttentionLayer builds with three slice copies and three head-split kernels
// (dnn/layers/multi_head_attention.cu:225-260); here TMA reads every head tile in place.
// It replaces upstream's matmul_kernel launches (:266-270, :283-287), SoftmaxLayer::forward
// (dnn/layers/softmax_layer.cu:26-81) and the head-merge kernel (:292-294), with the intended
// semantics (all batch-heads, scores = Q.K^T / sqrt(D)), not the launch bugs noted at :262-271.
//
// Softmax follows upstream exactly in form: p = exp(s + mask - rowmax) / (sum + 1e-6), and p = 0
// where mask < -1e8.  It is evaluated blockwise (online): per 128-key block the running row maximum
// and sum are updated and the block's probabilities multiply V on the tensor cores; the [T,T] score
// matrix never exists in memory.  The probabilities (scaled by a power of two) go to the tensor core as
// half-precision numbers — a single e4m3 rounding (3 mantissa bits) leaves ~2 % error on flat attention rows,
// outside the 1e-2 bound — so O += P.V is a kind::f16 product and each V tile is widened from its fp8 codes to
// halves (exactly) on its way: the exponentials run on packed halves (ex2.approx.f16x2, two keys per
// instruction) whose results are stored as they are, with no conversion.  The row sum is taken by the tensor
// core as well (P times a tile of ones), so it is the sum of exactly the values that multiply V.
//
// Work item = one (batch, head, 128-query block).  The grid is persistent: as many CTAs as fit on the GPU
// at once (two per SM at D = 64), each walking the items blockIdx.x, blockIdx.x + gridDim.x, ... with its
// barriers, TMEM and shared memory set up once; every barrier parity follows a running block counter.
// (Launched as one CTA per item, the block scheduler left the slot of a finished CTA empty for many
// microseconds: the kernel took 1.7x the sum of its CTA times.)
//   warp 0     TMA producer: an item's Q tile, then its K/V tiles through a 2-stage ring
//   warp 1     MMA issuer:   S = Q.K^T (kind::f8f6f4, M=128, N=128, K=D), O += P.V and row sums += P.1
//                            (kind::f16, M=128, N=D / 16, K=128)
//   warps 2-5  softmax:      one thread per query row with the block's 128 scores in registers (tcgen05.ld),
//                            row maximum, exp2 on packed halves stored straight into the swizzled fp16 A operand of
//                            the PV product; the same thread widens key row `row` of the block's V tile from fp8
//                            codes to the N-major fp16 B operand.  O and the row sum accumulate in TMEM across key
//                            blocks and are rescaled (tcgen05.ld/st) only when the row maximum has grown past a
//                            threshold.
//                            (Two threads per row with 64 scores each spilled at the 96 registers two CTAs per SM
//                            allow with 320 threads, and paid ~700 cycles per block to swap maxima; probabilities
//                            as the sum of two e4m3 numbers kept the PV product in fp8 but cost two fp8 packs per
//                            key on the conversion unit, which the exponentials already saturate: 94 us against
//                            82 us for this form at B=8 T=1024 H=12 D=64.)
// All mbarrier waits are bounded (status word, see df8_status_word_read).
#include "df8_internal.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

#include <atomic>
#include <cstdlib>

namespace df8 {

namespace {

using namespace ptx;

constexpr int kSoftmaxWarps = 4;  // one per TMEM lane quarter
constexpr int kAttnThreads = 64 + 32 * kSoftmaxWarps;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnArgs {
    const float* scale;  // {q, dq} of the QKV codes
    const float* mask;   // additive mask [mask_b,1,T,T] fp32 or null
    float* out;          // [B*T, E] fp32
    float* out_amax;     // 1 float or null
    int B, T, H, E;
    int n_qblk, n_items;
    int mask_mode;       // 0 none, 1 causal, 2 additive tensor
    int mask_b;
    int v_kind;          // fp8 kind of the QKV codes (how V widens to fp16)
    uint32_t idesc_qk, idesc_pv, idesc_sum;
    unsigned int* status;
};


template <int D>
struct AttnCfg {
    static constexpr int kQBytes = BQ * D;
    static constexpr int kKBytes = BKV * D;
    static constexpr int kStageBytes = 2 * kKBytes;  // K then V
    static constexpr int kStages = 2;
    static constexpr int kPBytes = 2 * BQ * 128;      // fp16 P [128 queries][128 keys]: two K atoms of 64 keys (128 B rows)
    static constexpr int kV16Bytes = BKV * D * 2;     // a block's V widened to fp16: [keys][D], D/64 atoms of 128 B rows
    static constexpr int kOnesBytes = 2 * 16 * 128;   // 16 x 128 tile of fp16 ones: B operand of the row-sum product
    static constexpr int kBarBytes = 128;  // mbarriers and the TMEM base slot
    static constexpr int kUsedBytes = kQBytes + kStages * kStageBytes + kPBytes + 2 * kV16Bytes + kOnesBytes + kBarBytes + 1024;
    // pad the request so that at most two CTAs share an SM: each allocates 256 of the 512 TMEM columns
    static constexpr int kSmemBytes = kUsedBytes < 110 * 1024 ? 110 * 1024 : kUsedBytes;
    // S: columns [0,128), O: [128, 128+D), row sum: [128+D, 128+D+16) (sixteen identical copies)
    static constexpr int kTmemCols = D == 64 ? 256 : 512;
};

__device__ __forceinline__ void record_timeout(unsigned int* status, unsigned int code) {
    if (status) {
        atomicCAS(status, 0u, code);
        atomicAdd(status + 1, 1u);
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// packed-half helpers: element 0 lives in the low half
__device__ __forceinline__ uint32_t pack_f16x2(float e0, float e1) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(e1), "f"(e0));
    return d;
}
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
    uint32_t d;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(d) : "r"(x));
    return d;
}
// ex2 pinned in program order between the barrier operations around it
__device__ __forceinline__ float ex2_ordered(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t f16x2_of_e4m3x2(uint32_t x) {
    uint32_t d;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"(static_cast<uint16_t>(x)));
    return d;
}
__device__ __forceinline__ uint32_t f16x2_of_e5m2x2(uint32_t x) {
    uint32_t d;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(d) : "h"(static_cast<uint16_t>(x)));
    return d;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, (D == 64 ? 2 : 1))
attention_fp8_kernel(const __grid_constant__ CUtensorMap tma_qkv, const AttnArgs args) {
    using Cfg = AttnCfg<D>;
    constexpr int SW = D;  // swizzle width of the Q/K/V tiles = their row length in bytes
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + Cfg::kQBytes;
    uint8_t* sP = sKV + Cfg::kStages * Cfg::kStageBytes;
    uint8_t* sV16 = sP + Cfg::kPBytes;
    uint8_t* sOnes = sV16 + 2 * Cfg::kV16Bytes;  // two V16 buffers: block x uses buffer x & 1
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOnes + Cfg::kOnesBytes);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;   // [2]
    uint64_t* kv_empty = bars + 3;  // [2]
    uint64_t* s_full = bars + 5;
    uint64_t* s_empty = bars + 6;
    uint64_t* p_full = bars + 7;
    uint64_t* o_full = bars + 8;
    uint64_t* q_empty = bars + 9;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    griddep_launch_dependents();
    const int T = args.T, E = args.E;
    const int n_items = args.n_items;
    const int n_kv_all = (T + BKV - 1) / BKV;
    // item -> (query block, head, batch).  Under the causal mask the query blocks are walked from the last
    // (longest key range) to the first, so that the short items fill the end of the schedule.
    struct Item {
        int qblk, h, b, n_kv;
    };
    auto decode = [&](int item) {
        Item it;
        const int hb = args.H * args.B;
        const int qr = item / hb, bh = item - qr * hb;
        it.qblk = args.mask_mode == 1 ? args.n_qblk - 1 - qr : qr;
        it.b = bh / args.H;
        it.h = bh - it.b * args.H;
        it.n_kv = n_kv_all;
        if (args.mask_mode == 1 && it.qblk + 1 < n_kv_all) it.n_kv = it.qblk + 1;  // blocks above the diagonal vanish
        return it;
    };

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(kv_full + s), 1);
            mbar_init(smem_u32(kv_empty + s), 1);
        }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(s_empty), kSoftmaxWarps);
        mbar_init(smem_u32(p_full), kSoftmaxWarps);
        mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(q_empty), 1);
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < Cfg::kOnesBytes / 4; i += kAttnThreads)
        reinterpret_cast<uint32_t*>(sOnes)[i] = 0x3C003C00u;  // fp16 1.0; every element equal, so no swizzle to honour
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    griddep_wait();  // set-up above overlaps the previous kernel's tail; global memory is touched below
    const uint32_t tmem_s = tmem_base;
    const uint32_t tmem_o = tmem_base + 128;
    const uint32_t tmem_l = tmem_base + 128 + D;

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tma_qkv);
            uint32_t kv_it = 0, item_it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
                const Item w = decode(item);
                const int row_base = w.b * T;
                // Q is single-buffered: the previous item's last Q.K^T must have read it
                if (item_it > 0 && !mbar_wait_bounded(smem_u32(q_empty), (item_it - 1) & 1)) {
                    record_timeout(args.status, 0x1000u);
                    break;
                }
                mbar_arrive_expect_tx(smem_u32(q_full), Cfg::kQBytes);
                tma_load_2d(smem_u32(sQ), &tma_qkv, smem_u32(q_full), w.h * D, row_base + w.qblk * BQ);
                for (int j = 0; j < w.n_kv; ++j, ++kv_it) {
                    const int s = kv_it & 1;
                    if (!mbar_wait_bounded(smem_u32(kv_empty + s), ((kv_it >> 1) & 1) ^ 1)) {
                        record_timeout(args.status, 0x1100u + s);
                        ok = false;
                        break;
                    }
                    uint8_t* st = sKV + s * Cfg::kStageBytes;
                    const uint32_t fb = smem_u32(kv_full + s);
                    mbar_arrive_expect_tx(fb, Cfg::kStageBytes);
                    tma_load_2d(smem_u32(st), &tma_qkv, fb, E + w.h * D, row_base + j * BKV);
                    tma_load_2d(smem_u32(st + Cfg::kKBytes), &tma_qkv, fb, 2 * E + w.h * D, row_base + j * BKV);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // The issuing thread's scalar instructions bound the MMA issue rate at these small shapes (about 5
            // cycles per dependent instruction, ~18 MMAs per key block), so every descriptor is split into a
            // constant high half and a low half that only needs 32-bit adds.
            const uint64_t qd = make_desc_kmajor<SW>(smem_u32(sQ));
            const uint64_t kd = make_desc_kmajor<SW>(smem_u32(sKV));
            // V16: N-major, 128-byte rows (64 halves of D) per key; a second N atom (D = 128) lies kV16Bytes / 2 further
            const uint64_t vd = make_desc_mnmajor<128>(smem_u32(sV16), Cfg::kV16Bytes / 2);
            const uint64_t pd = make_desc_kmajor<128>(smem_u32(sP));
            const uint64_t od = make_desc_kmajor<128>(smem_u32(sOnes));
            const uint32_t q_lo = desc_lo(qd), k_lo0 = desc_lo(kd), v_lo0 = desc_lo(vd), p_lo0 = desc_lo(pd), o_lo = desc_lo(od);
            const uint32_t qk_hi = desc_hi(qd), v_hi = desc_hi(vd), p_hi = desc_hi(pd);
            constexpr uint32_t kStageStep = Cfg::kStageBytes >> 4, kPAtomStep = (BQ * 128) >> 4, kOnesAtomStep = (16 * 128) >> 4;
            constexpr uint32_t kV16Step = Cfg::kV16Bytes >> 4;
            const uint32_t idesc_qk = args.idesc_qk, idesc_pv = args.idesc_pv, idesc_sum = args.idesc_sum;
            const uint32_t s_full_b = smem_u32(s_full), o_full_b = smem_u32(o_full);
            const uint32_t q_empty_b = smem_u32(q_empty);
            // S = Q.K^T of the block with running index x (its K/V stage is x & 1); `last`: the item's final
            // one, after which Q may be overwritten
            auto issue_qk = [&](uint32_t x, bool last) -> bool {
                if (!mbar_wait_bounded(smem_u32(kv_full + (x & 1)), (x >> 1) & 1)) return false;
                // the softmax warps release S as soon as they hold the previous block's scores in registers
                if (x > 0 && !mbar_wait_bounded(smem_u32(s_empty), (x - 1) & 1)) return false;
                tc_fence_after_sync();
                const uint32_t k_lo = k_lo0 + (x & 1) * kStageStep;
                tc_mma_f8(tmem_s, desc_join(q_lo, qk_hi), desc_join(k_lo, qk_hi), idesc_qk, 0);
#pragma unroll
                for (int k = 1; k < D / 32; ++k)
                    tc_mma_f8_acc(tmem_s, desc_join(q_lo + 2 * k, qk_hi), desc_join(k_lo + 2 * k, qk_hi), idesc_qk);
                tc_commit(s_full_b);
                if (last) tc_commit(q_empty_b);
                return true;
            };
            uint32_t g = 0, item_it = 0;  // g: running key-block counter over this CTA's items
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
                const Item w = decode(item);
                if (!mbar_wait_bounded(smem_u32(q_full), item_it & 1) || !issue_qk(g, w.n_kv == 1)) {
                    record_timeout(args.status, 0x1200u);
                    break;
                }
                for (int j = 0; j < w.n_kv; ++j) {
                    const uint32_t x = g + uint32_t(j), sj = x & 1;
                    // the next block's Q.K^T runs underneath this block's exponentials
                    if (j + 1 < w.n_kv && !issue_qk(x + 1, j + 2 == w.n_kv)) {
                        record_timeout(args.status, 0x1300u + (sj ^ 1));
                        ok = false;
                        break;
                    }
                    if (!mbar_wait_bounded(smem_u32(p_full), x & 1)) {
                        record_timeout(args.status, 0x1400u);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    // O (+)= P.V and row sums (+)= P.1, accumulated in TMEM over the item's key blocks; P = leading
                    // part + remainder.  Per 32 keys: P advances 32 bytes inside its 128-byte rows, V advances 32
                    // rows of D bytes.
                    // 16 keys per instruction: P advances 32 bytes inside its 128-byte rows (next K atom after four),
                    // V16 advances 16 rows of 128 bytes, the ones tile like P
                    const uint32_t v_lo = v_lo0 + sj * kV16Step;
                    if (j == 0) {
                        tc_mma_f16(tmem_o, desc_join(p_lo0, p_hi), desc_join(v_lo, v_hi), idesc_pv, 0);
                        tc_mma_f16(tmem_l, desc_join(p_lo0, p_hi), desc_join(o_lo, p_hi), idesc_sum, 0);
                    } else {
                        tc_mma_f16_acc(tmem_o, desc_join(p_lo0, p_hi), desc_join(v_lo, v_hi), idesc_pv);
                        tc_mma_f16_acc(tmem_l, desc_join(p_lo0, p_hi), desc_join(o_lo, p_hi), idesc_sum);
                    }
#pragma unroll
                    for (int k = 1; k < BKV / 16; ++k) {
                        const uint32_t pl = p_lo0 + (k / 4) * kPAtomStep + 2 * (k % 4);
                        tc_mma_f16_acc(tmem_o, desc_join(pl, p_hi), desc_join(v_lo + ((k * 16 * 128) >> 4), v_hi), idesc_pv);
                        tc_mma_f16_acc(tmem_l, desc_join(pl, p_hi),
                                       desc_join(o_lo + (k / 4) * kOnesAtomStep + 2 * (k % 4), p_hi), idesc_sum);
                    }
                    tc_commit(o_full_b);  // "P.V of block x done": P is free, O may be touched
                    tc_commit(smem_u32(kv_empty + sj));
                }
                g += uint32_t(w.n_kv);
            }
        }
    } else {
        const int q = warp & 3;            // TMEM lane quarter (warps w and w+4 share it)
        constexpr int HC = BKV;            // score columns per thread and block: the whole row
        const int row = q * 32 + lane;
        const float dq = ld_l2_f32(args.scale + 1);
        const float cs = dq * dq * rsqrtf(float(D)) * kLog2e;  // raw score -> log2 domain
        const uint32_t lane_addr = uint32_t(q * 32) << 16;

        // Probabilities are formed as p' = 2^kPShift * exp2(t - m) against a reference maximum m that is only
        // moved (and O, l rescaled) when the true running maximum has grown by more than kLazy: then
        // p' <= 2^(kPShift + kLazy) stays inside e4m3 (max 448), and the TMEM round trip that rescales O
        // is rare after the first key blocks.
        // The exponent t - m + kPShift is rounded to half precision before exp2: its magnitude stays below 8
        // for every key that matters, i.e. an absolute error of at most 2^-9 in the exponent (0.14 % of p).
        constexpr float kPShift = 5.0f;
        constexpr float kLazy = 2.5f;
        bool ok = true;
        int pv_waited = 0;  // number of "P.V done" phases this thread has observed (over all items)
        int g = 0;          // running key-block counter over this CTA's items
        float amax = 0.f;   // max|out| over this thread's outputs of all items

        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const Item w = decode(item);
        const int n_kv = w.n_kv, h = w.h, b = w.b;
        const int q0 = w.qblk * BQ, row_base = b * T;
        const int qi = q0 + row;
        const float* mrow = nullptr;
        if (args.mask_mode == 2 && qi < T)
            mrow = args.mask + (size_t(args.mask_b > 1 ? b : 0) * T + qi) * T;
        float m = -INFINITY;       // reference maximum of the exponentials (log2 domain)
        float m_true = -INFINITY;  // true running maximum of the row

        for (int j = 0; j < n_kv; ++j) {
            const int gj = g + j;
            const int k0 = j * BKV;
            // ---- V: fp8 codes -> halves (exact), key `row` of the block per thread, into the N-major fp16 tile.
            // Done first: the V tile lands with the K tile, before S can be ready, and V16 buffer gj & 1 was last read
            // by the P.V of block gj - 2, which the previous block's wait (before its P stores) has seen complete ----
            if (!mbar_wait_bounded(smem_u32(kv_full + (gj & 1)), (gj >> 1) & 1)) {
                if (lane == 0) record_timeout(args.status, 0x1c00u);
                ok = false;
                break;
            }
            {
                const uint8_t* vsrc = sKV + (gj & 1) * Cfg::kStageBytes + Cfg::kKBytes + row * D;
                uint8_t* vdst = sV16 + (gj & 1) * Cfg::kV16Bytes + row * 128;
                const int sw_in = (D == 64) ? ((row >> 1) & 3) : (row & 7);  // TMA swizzle of the D-byte source rows
                const bool e4m3 = args.v_kind == DF8_E4M3;
#pragma unroll
                for (int c = 0; c < D / 16; ++c) {
                    const uint4 in = *reinterpret_cast<const uint4*>(vsrc + ((c ^ sw_in) << 4));
                    const uint32_t wds[4] = {in.x, in.y, in.z, in.w};
                    uint32_t h[8];
                    if (e4m3) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            h[2 * k] = f16x2_of_e4m3x2(wds[k] & 0xFFFFu);
                            h[2 * k + 1] = f16x2_of_e4m3x2(wds[k] >> 16);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            h[2 * k] = f16x2_of_e5m2x2(wds[k] & 0xFFFFu);
                            h[2 * k + 1] = f16x2_of_e5m2x2(wds[k] >> 16);
                        }
                    }
                    // 16 codes -> 32 bytes = chunks 2c, 2c+1 of the key's 128-byte rows (one row per 64 values of D)
                    uint8_t* vrow = vdst + ((2 * c) >> 3) * (Cfg::kV16Bytes / 2);
                    const int k0c = (2 * c) & 7;
                    *reinterpret_cast<uint4*>(vrow + ((k0c ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(vrow + (((k0c + 1) ^ (row & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
                }
            }
            if (!mbar_wait_bounded(smem_u32(s_full), gj & 1)) {
                if (lane == 0) record_timeout(args.status, 0x1500u);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            // this row's 128 scores into registers, then S is released at once
            uint32_t r[HC];
#pragma unroll
            for (int c = 0; c < HC / 32; ++c)
                tmem_ld_32x32(tmem_s + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(s_empty));

            const bool edge = (j * BKV + BKV > T) || (args.mask_mode == 1 && j * BKV + BKV - 1 > q0) || (args.mask_mode == 2);
            float mb = -INFINITY;
            if (!edge) {
                float ra = -INFINITY, rb = -INFINITY, rc = -INFINITY, rd = -INFINITY;  // four dependency chains
#pragma unroll
                for (int i = 0; i < HC; i += 8) {
                    ra = fmax3(ra, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    rb = fmax3(rb, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    rc = fmax3(rc, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                    rd = fmax3(rd, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                }
                mb = fmaxf(fmaxf(ra, rb), fmaxf(rc, rd)) * cs;  // cs > 0: the maximum commutes with the scaling; r stays unscaled (see below)
            } else {
#pragma unroll
                for (int i = 0; i < HC; ++i) {
                    const int kj = k0 + i;
                    float t = __uint_as_float(r[i]) * cs;
                    if (kj >= T || (args.mask_mode == 1 && kj > qi)) {
                        t = -INFINITY;
                    } else if (mrow) {
                        const float mv = mrow[kj];
                        t = (mv < -1e8f) ? -INFINITY : fmaf(mv, kLog2e, t);
                    }
                    r[i] = __float_as_uint(t);
                    mb = fmaxf(mb, t);
                }
            }
            m_true = fmaxf(m_true, mb);

            // move the reference maximum?  (always on the first block that has an unmasked key)
            const bool move = m_true > m + kLazy;  // also true while m is -inf and m_true is finite
            if (__any_sync(0xffffffffu, move)) {
                float alpha = 1.f;
                if (move) {
                    alpha = ex2(m - m_true);  // 0 when m was -inf
                    m = m_true;
                }
                if (j > 0) {
                    // O holds the products of blocks < j: wait until the last of them has landed, then scale
                    // this row
                    while (pv_waited < gj) {
                        if (!mbar_wait_bounded(smem_u32(o_full), pv_waited & 1)) {
                            ok = false;
                            break;
                        }
                        ++pv_waited;
                    }
                    if (!__all_sync(0xffffffffu, ok)) {
                        if (lane == 0) record_timeout(args.status, 0x1600u);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < D / 16; ++c) {  // small pieces: the row's 128 scores stay in registers meanwhile
                        uint32_t o[16];
                        const uint32_t oaddr = tmem_o + lane_addr + c * 16;
                        tmem_ld_32x16(oaddr, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x16(oaddr, o);
                    }
                    {  // the row sum: only column 0 of its sixteen copies is ever read back
                        const uint32_t laddr = tmem_l + lane_addr;
                        const float lv = __uint_as_float(tmem_ld_32x1(laddr));
                        tmem_ld_wait();
                        tmem_st_32x1(laddr, __float_as_uint(lv * alpha));
                    }
                    tmem_st_wait();
                }
            }
            const float shift = ((m == -INFINITY) ? 0.f : m) - kPShift;
            const float ecs = edge ? 1.f : cs;  // masked blocks hold scores already scaled (and masked) in r

            // ---- P = 2^(t - m + kPShift) as halves: all 64 packed results first, the stores after the wait below ----
            const float nshift = -shift;
            uint32_t w[HC / 2];
#pragma unroll
            for (int g = 0; g < HC / 2; ++g)
                w[g] = ex2_f16x2(pack_f16x2(fmaf(__uint_as_float(r[2 * g]), ecs, nshift),
                                            fmaf(__uint_as_float(r[2 * g + 1]), ecs, nshift)));
            // P is a single buffer: the P.V of the previous block must have read it.  That product was issued at
            // the end of the previous block's softmax and has had this whole block's arithmetic to finish.
            while (pv_waited < gj) {
                if (!mbar_wait_bounded(smem_u32(o_full), pv_waited & 1)) {
                    ok = false;
                    break;
                }
                ++pv_waited;
            }
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) record_timeout(args.status, 0x1700u);
                ok = false;
                break;
            }
            // 64 keys (128 bytes) per K atom; 32 keys = 64 bytes = four 16-byte chunks
            uint8_t* prow = sP + row * 128;
#pragma unroll
            for (int c = 0; c < HC / 32; ++c) {
                uint8_t* patom = prow + (c >> 1) * (BQ * 128);
                const int cb = (c & 1) * 4;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    *reinterpret_cast<uint4*>(patom + (((cb + k) ^ (row & 7)) << 4)) =
                        make_uint4(w[16 * c + 4 * k], w[16 * c + 4 * k + 1], w[16 * c + 4 * k + 2], w[16 * c + 4 * k + 3]);
            }

            tc_fence_before_sync();  // orders the O rescale (if any) before the issuer's next P.V
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(p_full));
        }

        if (ok) {
            while (pv_waited < g + n_kv) {
                if (!mbar_wait_bounded(smem_u32(o_full), pv_waited & 1)) {
                    ok = false;
                    break;
                }
                ++pv_waited;
            }
            if (!ok && lane == 0) record_timeout(args.status, 0x1800u);
        }
        if (!__all_sync(0xffffffffu, ok)) break;
        {
            tc_fence_after_sync();
            // the row sum, accumulated by the tensor core next to O
            float l = 0.f;
            if (n_kv > 0) {
                l = __uint_as_float(tmem_ld_32x1(tmem_l + lane_addr));
                tmem_ld_wait();
            }
            // upstream: p = exp(s - max) / (sum + 1e-6).  Here sum' = 2^kPShift * sum * 2^(max - m), so the
            // 1e-6 is carried over with the same factor.
            const float eps = 1e-6f * ex2(kPShift + ((m == -INFINITY) ? 0.f : (m_true - m)));
            const float inv = dq / (l + eps);
            // Rows leave through shared memory so that global stores are whole 128-byte row segments: the
            // staging area is this warp's own 32 rows of the first P buffer, idle once the item's last P.V is done
            // and not touched by the other warps (they only ever write their own rows).
            uint8_t* stg = sP + q * 32 * 128;
            float* obase = args.out + (size_t(row_base) + q0 + q * 32) * E + h * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int d = 0; d < 32; d += 4) {
                    float4 f = make_float4(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv,
                                           __uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                    if (l == 0.f) f = make_float4(0.f, 0.f, 0.f, 0.f);  // every key masked: zeros, as upstream
                    if (qi < T) amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
                    *reinterpret_cast<float4*>(stg + lane * 128 + (((d >> 2) ^ (lane & 7)) << 4)) = f;
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3), k = lane & 7;
                    const float4 f = *reinterpret_cast<const float4*>(stg + rr * 128 + ((k ^ (rr & 7)) << 4));
                    if (q0 + q * 32 + rr < T) *reinterpret_cast<float4*>(obase + size_t(rr) * E + c * 32 + k * 4) = f;
                }
                __syncwarp();
            }
            tc_fence_before_sync();  // O and the row sum are in registers before this warp's next p_full arrival
        }
        g += n_kv;
        }  // items
        if (args.out_amax) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---- two query tiles per CTA (D = 64, T a multiple of 256) ---------------------------------------------------
//
// Clock stamps of the kernel above (B = 8, T = 1024, H = 12): a key block costs each softmax warp ~4.9 k cycles
// (V widening 0.7 k, TMEM load 0.25 k, row maximum 0.7 k, exponentials 1.8 k, P stores and barrier traffic
// 0.9 k) of which the special-function unit needs 1 k, and the row-sum products cost the tensor core as much issue
// time as P.V itself.  This variant keeps one CTA per SM with two 128-query tiles of the same (batch, head):
//   * each K/V tile is loaded once for both query tiles, and its V is widened to halves by two warps of their
//     own, off the softmax warps' chain;
//   * the B operand of P.V is the V tile plus an atom of ones (N = 80): columns 64..79 of O are the row sums,
//     no separate row-sum product;
//   * the K/V ring has three stages;
//   * the two tiles take turns at the exponentials.  Left alone they run in lockstep (the MMA warp serves both in
//     one loop) and their softmax warps — the two on a scheduler hold the same lane quarter of the two tiles — hit
//     the special-function unit together: 2.25 k cycles for a block's exponentials instead of 1.25 k, with the
//     unit idle for the rest of the block.  One mbarrier per tile and lane quarter orders them: tile 1 starts the
//     exponentials of block x when tile 0 has issued half of those of block x, tile 0 those of block x + 1 when
//     tile 1 has issued half of those of block x; everything else (TMEM loads, maxima, P stores, waits) overlaps
//     the other tile's turn.  (One warp alone does not fill the unit, hence the hand-over at half.)
//   * exp2 is evaluated in fp32 and the results packed to halves: as fast here as ex2 on packed halves, and the
//     exponent is not rounded to half precision first.
// (Two threads per query row — sixteen softmax warps with 64 scores each — was measured as well: the halves of
// a row must agree on the reference maximum every key block, and that exchange (~700 cycles per block through
// shared memory and an mbarrier) cost more than the shorter phases saved: 91 us against 79 us.)
//   warp 0      TMA producer: Q (both tiles) per item, K/V codes through the ring
//   warp 1      MMA issuer: S_t = Q_t.K^T for both tiles one key block ahead, O_t (+)= P_t.[V | 1]
//   warps 2-9   softmax: warp w -> TMEM lane quarter w % 4, tile (w - 2) / 4; one thread per query row
//   warps 10-11 V widening: two keys per thread and key block
constexpr int kWideSoftmaxWarps = 8;
constexpr int kWideWidenWarps = 2;
constexpr int kWideThreads = 64 + 32 * (kWideSoftmaxWarps + kWideWidenWarps);

struct WideCfg {
    static constexpr int D = 64;
    static constexpr int kQBytes = 2 * BQ * D;       // both query tiles
    static constexpr int kKBytes = BKV * D;
    static constexpr int kStageBytes = 2 * kKBytes;  // K codes then V codes
    static constexpr int kStages = 3;
    static constexpr int kPBytes = 2 * BQ * 128;     // fp16 P of one tile: two K atoms of 64 keys
    static constexpr int kV16Bytes = BKV * D * 2;    // fp16 V: [keys][64 halves]
    static constexpr int kVBufBytes = 2 * kV16Bytes; // ... followed by an equally large N atom of ones
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes =
        kQBytes + kStages * kStageBytes + 2 * kPBytes + 2 * kVBufBytes + kBarBytes + 1024;
    static constexpr int kTmemCols = 512;  // tile t: S at 256 t (128 columns), O and row sums at 256 t + 128 (80 columns)
    static constexpr int kON = D + 16;     // N of the P.[V | 1] product
};
static_assert(WideCfg::kSmemBytes <= 227 * 1024, "shared memory budget");

__global__ void __launch_bounds__(kWideThreads, 1)
attention_fp8_wide_kernel(const __grid_constant__ CUtensorMap tma_qkv, const AttnArgs args) {
    using Cfg = WideCfg;
    constexpr int D = Cfg::D;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + Cfg::kQBytes;
    uint8_t* sP = sKV + Cfg::kStages * Cfg::kStageBytes;  // tile t at sP + t * kPBytes
    uint8_t* sV = sP + 2 * Cfg::kPBytes;                  // buffer b at sV + b * kVBufBytes: V16 then ones
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * Cfg::kVBufBytes);
    uint64_t* q_full = bars;
    uint64_t* q_empty = bars + 1;
    uint64_t* kv_full = bars + 2;     // [3]
    uint64_t* kv_empty = bars + 5;    // [3]  the block's Q.K^T products done (1) and its V widened (2 warps)
    uint64_t* v16_full = bars + 8;    // [2]  the widening warps
    uint64_t* v16_empty = bars + 10;  // [2]  the P.V products that read the buffer are done
    uint64_t* s_full = bars + 12;     // [2 tiles]
    uint64_t* s_empty = bars + 14;    // [2]  the tile's 4 softmax warps
    uint64_t* p_full = bars + 16;     // [2]  the tile's 4 softmax warps
    uint64_t* o_full = bars + 18;     // [2]
    uint64_t* turn = bars + 20;       // [2 tiles][4 quarters]: "the other tile's warp of this quarter has issued its exponentials"
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 28);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    griddep_launch_dependents();
    const int T = args.T, E = args.E;
    const int n_items = args.n_items;
    const int n_kv_all = T / BKV;
    const int n_pairs = T / (2 * BQ);
    struct Item {
        int pair, h, b, n_kv[2], n_max;
    };
    auto decode = [&](int item) {
        Item it;
        const int hb = args.H * args.B;
        const int pr = item / hb, bh = item - pr * hb;
        it.pair = args.mask_mode == 1 ? n_pairs - 1 - pr : pr;  // causal: longest key ranges first
        it.b = bh / args.H;
        it.h = bh - it.b * args.H;
        it.n_kv[0] = it.n_kv[1] = n_kv_all;
        if (args.mask_mode == 1) {  // blocks above the diagonal vanish
            it.n_kv[0] = 2 * it.pair + 1;
            it.n_kv[1] = 2 * it.pair + 2;
        }
        it.n_max = it.n_kv[1];
        return it;
    };

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        mbar_init(smem_u32(q_empty), 1);
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(smem_u32(kv_full + s), 1);
            mbar_init(smem_u32(kv_empty + s), 1 + kWideWidenWarps);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(v16_full + i), kWideWidenWarps);
            mbar_init(smem_u32(v16_empty + i), 1);
            mbar_init(smem_u32(s_full + i), 1);
            mbar_init(smem_u32(s_empty + i), kWideSoftmaxWarps / 2);
            mbar_init(smem_u32(p_full + i), kWideSoftmaxWarps / 2);
            mbar_init(smem_u32(o_full + i), 1);
        }
        for (int i = 0; i < 8; ++i) mbar_init(smem_u32(turn + i), 1);
        mbar_fence_init();
    }
    for (int b = 0; b < 2; ++b) {  // the atoms of ones: every element equal, so no swizzle to honour
        uint32_t* ones = reinterpret_cast<uint32_t*>(sV + b * Cfg::kVBufBytes + Cfg::kV16Bytes);
        for (int i = threadIdx.x; i < Cfg::kV16Bytes / 4; i += kWideThreads) ones[i] = 0x3C003C00u;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    griddep_wait();

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tma_qkv);
            uint32_t stage = 0, phase = 0, item_it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
                const Item w = decode(item);
                const int row_base = w.b * T;
                if (item_it > 0 && !mbar_wait_bounded(smem_u32(q_empty), (item_it - 1) & 1)) {
                    record_timeout(args.status, 0x3000u);
                    break;
                }
                mbar_arrive_expect_tx(smem_u32(q_full), Cfg::kQBytes);
                tma_load_2d(smem_u32(sQ), &tma_qkv, smem_u32(q_full), w.h * D, row_base + w.pair * 2 * BQ);
                tma_load_2d(smem_u32(sQ + BQ * D), &tma_qkv, smem_u32(q_full), w.h * D, row_base + w.pair * 2 * BQ + BQ);
                for (int j = 0; j < w.n_max; ++j) {
                    if (!mbar_wait_bounded(smem_u32(kv_empty + stage), phase ^ 1)) {
                        record_timeout(args.status, 0x3100u + stage);
                        ok = false;
                        break;
                    }
                    uint8_t* st = sKV + stage * Cfg::kStageBytes;
                    const uint32_t fb = smem_u32(kv_full + stage);
                    mbar_arrive_expect_tx(fb, Cfg::kStageBytes);
                    tma_load_2d(smem_u32(st), &tma_qkv, fb, E + w.h * D, row_base + j * BKV);
                    tma_load_2d(smem_u32(st + Cfg::kKBytes), &tma_qkv, fb, 2 * E + w.h * D, row_base + j * BKV);
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint64_t qd = make_desc_kmajor<D>(smem_u32(sQ));
            const uint64_t kd = make_desc_kmajor<D>(smem_u32(sKV));
            const uint64_t vd = make_desc_mnmajor<128>(smem_u32(sV), Cfg::kV16Bytes);  // second N atom: the ones
            const uint64_t pd = make_desc_kmajor<128>(smem_u32(sP));
            const uint32_t q_lo0 = desc_lo(qd), k_lo0 = desc_lo(kd), v_lo0 = desc_lo(vd), p_lo0 = desc_lo(pd);
            const uint32_t qk_hi = desc_hi(qd), v_hi = desc_hi(vd), p_hi = desc_hi(pd);
            constexpr uint32_t kStageStep = Cfg::kStageBytes >> 4, kPAtomStep = (BQ * 128) >> 4;
            constexpr uint32_t kVBufStep = Cfg::kVBufBytes >> 4, kPTileStep = Cfg::kPBytes >> 4, kQTileStep = (BQ * D) >> 4;
            const uint32_t idesc_qk = args.idesc_qk, idesc_pv = args.idesc_pv;
            uint32_t g[2] = {0, 0};      // running key-block counters of the two tiles
            uint32_t kvc = 0;            // running counter of loaded key blocks: V16 buffer kvc & 1
            uint32_t stage = 0, phase = 0;  // ring position of the block whose Q.K^T is issued next
            uint32_t item_it = 0;
            bool ok = true;
            // S_t = Q_t.K^T for the key block in ring slot (stage, phase), for the tiles that still have blocks
            auto issue_qk = [&](const Item& w, int xq) -> bool {
                if (!mbar_wait_bounded(smem_u32(kv_full + stage), phase)) return false;
                for (int t = 0; t < 2; ++t) {
                    if (xq >= w.n_kv[t]) continue;
                    const uint32_t gx = g[t] + uint32_t(xq);
                    // the tile's softmax warps release S once the previous block's scores are in registers
                    if (gx > 0 && !mbar_wait_bounded(smem_u32(s_empty + t), (gx - 1) & 1)) return false;
                    tc_fence_after_sync();
                    const uint32_t tmem_s = tmem_base + 256 * t;
                    const uint32_t q_lo = q_lo0 + t * kQTileStep, k_lo = k_lo0 + stage * kStageStep;
                    tc_mma_f8(tmem_s, desc_join(q_lo, qk_hi), desc_join(k_lo, qk_hi), idesc_qk, 0);
                    tc_mma_f8_acc(tmem_s, desc_join(q_lo + 2, qk_hi), desc_join(k_lo + 2, qk_hi), idesc_qk);
                    tc_commit(smem_u32(s_full + t));
                }
                tc_commit(smem_u32(kv_empty + stage));  // the K codes of this slot are no longer needed
                if (xq + 1 == w.n_max) tc_commit(smem_u32(q_empty));
                if (++stage == Cfg::kStages) {
                    stage = 0;
                    phase ^= 1;
                }
                return true;
            };
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_it) {
                const Item w = decode(item);
                if (!mbar_wait_bounded(smem_u32(q_full), item_it & 1) || !issue_qk(w, 0)) {
                    record_timeout(args.status, 0x3200u);
                    break;
                }
                for (int x = 0; x < w.n_max && ok; ++x) {
                    if (x + 1 < w.n_max && !issue_qk(w, x + 1)) {
                        record_timeout(args.status, 0x3300u);
                        ok = false;
                        break;
                    }
                    const uint32_t kx = kvc + uint32_t(x), vb = kx & 1;
                    if (!mbar_wait_bounded(smem_u32(v16_full + vb), (kx >> 1) & 1)) {
                        record_timeout(args.status, 0x3400u);
                        ok = false;
                        break;
                    }
                    const uint32_t v_lo = v_lo0 + vb * kVBufStep;
                    for (int t = 0; t < 2; ++t) {
                        if (x >= w.n_kv[t]) continue;
                        if (!mbar_wait_bounded(smem_u32(p_full + t), (g[t] + uint32_t(x)) & 1)) {
                            record_timeout(args.status, 0x3500u + t);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t tmem_o = tmem_base + 256 * t + 128;
                        const uint32_t p_lo = p_lo0 + t * kPTileStep;
                        // 16 keys per instruction: P advances 32 bytes inside its 128-byte rows (next K atom after
                        // four), V16 and the ones advance 16 rows of 128 bytes
                        if (x == 0) tc_mma_f16(tmem_o, desc_join(p_lo, p_hi), desc_join(v_lo, v_hi), idesc_pv, 0);
                        else tc_mma_f16_acc(tmem_o, desc_join(p_lo, p_hi), desc_join(v_lo, v_hi), idesc_pv);
#pragma unroll
                        for (int k = 1; k < BKV / 16; ++k)
                            tc_mma_f16_acc(tmem_o, desc_join(p_lo + (k / 4) * kPAtomStep + 2 * (k % 4), p_hi),
                                           desc_join(v_lo + ((k * 16 * 128) >> 4), v_hi), idesc_pv);
                        tc_commit(smem_u32(o_full + t));  // "P_t.V of this block done": P_t is free, O_t may be touched
                    }
                    if (ok) tc_commit(smem_u32(v16_empty + vb));
                }
                g[0] += uint32_t(w.n_kv[0]);
                g[1] += uint32_t(w.n_kv[1]);
                kvc += uint32_t(w.n_max);
            }
        }
    } else if (warp >= 2 + kWideSoftmaxWarps) {
        // ---- V: fp8 codes -> halves (exact) into the N-major fp16 tile, two keys per thread ----
        const int wid = (warp - 2 - kWideSoftmaxWarps) * 32 + lane;
        uint32_t stage = 0, phase = 0, kx = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const Item w = decode(item);
            for (int x = 0; x < w.n_max; ++x, ++kx) {
                const uint32_t vb = kx & 1;
                // the tile has landed, and the P.V products of block kx - 2 have read this V16 buffer
                if (!mbar_wait_bounded(smem_u32(kv_full + stage), phase) ||
                    (kx >= 2 && !mbar_wait_bounded(smem_u32(v16_empty + vb), ((kx - 2) >> 1) & 1))) {
                    if (lane == 0) record_timeout(args.status, 0x3600u);
                    ok = false;
                    break;
                }
                const bool e4m3 = args.v_kind == DF8_E4M3;
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const int key = 2 * wid + kk;
                    const uint8_t* vsrc = sKV + stage * Cfg::kStageBytes + Cfg::kKBytes + key * D;
                    uint8_t* vrow = sV + vb * Cfg::kVBufBytes + key * 128;
                    const int sw_in = (key >> 1) & 3;  // TMA swizzle of the 64-byte source rows
#pragma unroll
                    for (int c = 0; c < D / 16; ++c) {
                        const uint4 in = *reinterpret_cast<const uint4*>(vsrc + ((c ^ sw_in) << 4));
                        const uint32_t wds[4] = {in.x, in.y, in.z, in.w};
                        uint32_t hv[8];
                        if (e4m3) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                hv[2 * k] = f16x2_of_e4m3x2(wds[k] & 0xFFFFu);
                                hv[2 * k + 1] = f16x2_of_e4m3x2(wds[k] >> 16);
                            }
                        } else {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                hv[2 * k] = f16x2_of_e5m2x2(wds[k] & 0xFFFFu);
                                hv[2 * k + 1] = f16x2_of_e5m2x2(wds[k] >> 16);
                            }
                        }
                        *reinterpret_cast<uint4*>(vrow + (((2 * c) ^ (key & 7)) << 4)) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
                        *reinterpret_cast<uint4*>(vrow + (((2 * c + 1) ^ (key & 7)) << 4)) = make_uint4(hv[4], hv[5], hv[6], hv[7]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(v16_full + vb));
                    mbar_arrive(smem_u32(kv_empty + stage));
                }
                if (++stage == Cfg::kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else {
        const int sw = warp - 2;
        const int q = warp & 3;         // TMEM lane quarter
        const int t = sw >> 2;          // query tile
        const int row = q * 32 + lane;  // query row within the tile
        const float dq = ld_l2_f32(args.scale + 1);
        const float cs = dq * dq * rsqrtf(float(D)) * kLog2e;
        const uint32_t lane_addr = uint32_t(q * 32) << 16;
        const uint32_t tmem_s = tmem_base + 256 * t;
        const uint32_t tmem_o = tmem_base + 256 * t + 128;
        uint8_t* sPt = sP + t * Cfg::kPBytes;
        constexpr float kPShift = 5.0f;
        constexpr float kLazy = 2.5f;
        constexpr int HC = BKV;  // score columns per thread and block: the whole row
        constexpr int kTurnAt = HC / 4;  // pairs of exponentials issued when the other tile may start its own
        bool ok = true;
        uint32_t pv_waited = 0;  // "P_t.V done" phases this thread has observed
        uint32_t gt = 0;         // running key-block counter of this thread's tile
        uint32_t go = 0;         // ... and of the other tile
        const uint32_t my_turn = smem_u32(turn + t * 4 + q), other_turn = smem_u32(turn + (t ^ 1) * 4 + q);
        float amax = 0.f;

        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const Item w = decode(item);
            const int n_t = w.n_kv[t], n_o = w.n_kv[t ^ 1];
            const int h = w.h, b = w.b;
            const int q0 = (2 * w.pair + t) * BQ, row_base = b * T;
            const int qi = q0 + row;
            const float* mrow = nullptr;
            if (args.mask_mode == 2) mrow = args.mask + (size_t(args.mask_b > 1 ? b : 0) * T + qi) * T;
            float m = -INFINITY;       // reference maximum of the exponentials (log2 domain)
            float m_true = -INFINITY;  // true running maximum of the row

            for (int x = 0; x < n_t; ++x) {
                const uint32_t gj = gt + uint32_t(x);
                const int k0 = x * BKV;
                if (!mbar_wait_bounded(smem_u32(s_full + t), gj & 1)) {
                    if (lane == 0) record_timeout(args.status, 0x3700u);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t r[HC];
#pragma unroll
                for (int c = 0; c < HC / 32; ++c)
                    tmem_ld_32x32(tmem_s + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(s_empty + t));

                const bool edge = (args.mask_mode == 1 && x * BKV + BKV - 1 > q0) || (args.mask_mode == 2);
                float mb = -INFINITY;
                if (!edge) {
                    float ra = -INFINITY, rb = -INFINITY, rc = -INFINITY, rd = -INFINITY;
#pragma unroll
                    for (int i = 0; i < HC; i += 8) {
                        ra = fmax3(ra, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                        rb = fmax3(rb, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                        rc = fmax3(rc, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                        rd = fmax3(rd, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                    }
                    mb = fmaxf(fmaxf(ra, rb), fmaxf(rc, rd)) * cs;
                } else {
#pragma unroll
                    for (int i = 0; i < HC; ++i) {
                        const int kj = k0 + i;
                        float tv = __uint_as_float(r[i]) * cs;
                        if (args.mask_mode == 1 && kj > qi) {
                            tv = -INFINITY;
                        } else if (mrow) {
                            const float mv = mrow[kj];
                            tv = (mv < -1e8f) ? -INFINITY : fmaf(mv, kLog2e, tv);
                        }
                        r[i] = __float_as_uint(tv);
                        mb = fmaxf(mb, tv);
                    }
                }
                m_true = fmaxf(m_true, mb);

                const bool move = m_true > m + kLazy;  // also true while m is -inf and m_true is finite
                if (__any_sync(0xffffffffu, move)) {
                    float alpha = 1.f;
                    if (move) {
                        alpha = ex2(m - m_true);
                        m = m_true;
                    }
                    if (x > 0) {
                        while (pv_waited < gj) {
                            if (!mbar_wait_bounded(smem_u32(o_full + t), pv_waited & 1)) {
                                ok = false;
                                break;
                            }
                            ++pv_waited;
                        }
                        if (!__all_sync(0xffffffffu, ok)) {
                            if (lane == 0) record_timeout(args.status, 0x3900u);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int c = 0; c < D / 16; ++c) {  // small pieces: the scores stay in registers meanwhile
                            uint32_t o[16];
                            const uint32_t oaddr = tmem_o + lane_addr + c * 16;
                            tmem_ld_32x16(oaddr, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st_32x16(oaddr, o);
                        }
                        {  // the row sum: only column 64 of its sixteen copies is ever read back
                            const uint32_t laddr = tmem_o + lane_addr + D;
                            const float lv = __uint_as_float(tmem_ld_32x1(laddr));
                            tmem_ld_wait();
                            tmem_st_32x1(laddr, __float_as_uint(lv * alpha));
                        }
                        tmem_st_wait();
                    }
                }
                const float nshift = kPShift - ((m == -INFINITY) ? 0.f : m);
                const float ecs = edge ? 1.f : cs;

                // this tile's turn at the special-function unit: tile 0 waits for tile 1's block x - 1, tile 1 for
                // tile 0's block x (which under the causal mask may not exist: tile 0 has one block less)
                if (t == 0 ? x > 0 : x < n_o) {
                    const uint32_t need = t == 0 ? go + uint32_t(x) - 1 : go + uint32_t(x);  // arrival number, from 0
                    if (!mbar_wait_bounded(my_turn, need & 1)) {
                        if (lane == 0) record_timeout(args.status, 0x3c00u);
                        ok = false;
                        break;
                    }
                }
                uint32_t pw[HC / 2];
#pragma unroll
                for (int i = 0; i < HC / 2; ++i) {
                    pw[i] = pack_f16x2(ex2_ordered(fmaf(__uint_as_float(r[2 * i]), ecs, nshift)),
                                       ex2_ordered(fmaf(__uint_as_float(r[2 * i + 1]), ecs, nshift)));
                    if (i == kTurnAt - 1 && lane == 0) mbar_arrive(other_turn);
                }
                // P_t is a single buffer: the tile's previous P.V must have read it
                while (pv_waited < gj) {
                    if (!mbar_wait_bounded(smem_u32(o_full + t), pv_waited & 1)) {
                        ok = false;
                        break;
                    }
                    ++pv_waited;
                }
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) record_timeout(args.status, 0x3a00u);
                    ok = false;
                    break;
                }
                // 64 keys (128 bytes) per K atom
                uint8_t* prow = sPt + row * 128;
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) {
                    uint8_t* patom = prow + (c >> 1) * (BQ * 128);
                    const int cb = (c & 1) * 4;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        *reinterpret_cast<uint4*>(patom + (((cb + k) ^ (row & 7)) << 4)) =
                            make_uint4(pw[16 * c + 4 * k], pw[16 * c + 4 * k + 1], pw[16 * c + 4 * k + 2], pw[16 * c + 4 * k + 3]);
                }
                tc_fence_before_sync();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(p_full + t));
            }
            if (!__all_sync(0xffffffffu, ok)) break;

            while (pv_waited < gt + uint32_t(n_t)) {
                if (!mbar_wait_bounded(smem_u32(o_full + t), pv_waited & 1)) {
                    ok = false;
                    break;
                }
                ++pv_waited;
            }
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) record_timeout(args.status, 0x3b00u);
                break;
            }
            {
                tc_fence_after_sync();
                const float l = __uint_as_float(tmem_ld_32x1(tmem_o + lane_addr + D));
                tmem_ld_wait();
                // upstream: p = exp(s - max) / (sum + 1e-6); the sums here carry 2^kPShift * 2^(max - m)
                const float eps = 1e-6f * ex2(kPShift + ((m == -INFINITY) ? 0.f : (m_true - m)));
                const float inv = dq / (l + eps);
                // rows leave through this warp's own 32 rows of the tile's first P atom, idle once the item's last
                // P.V is done, so that global stores are whole 128-byte row segments
                uint8_t* stg = sPt + q * 32 * 128;
                float* obase = args.out + (size_t(row_base) + q0 + q * 32) * E + h * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int d = 0; d < 32; d += 4) {
                        float4 f = make_float4(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv,
                                               __uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                        if (l == 0.f) f = make_float4(0.f, 0.f, 0.f, 0.f);  // every key masked: zeros, as upstream
                        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
                        *reinterpret_cast<float4*>(stg + lane * 128 + (((d >> 2) ^ (lane & 7)) << 4)) = f;
                    }
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3), k = lane & 7;
                        const float4 f = *reinterpret_cast<const float4*>(stg + rr * 128 + ((k ^ (rr & 7)) << 4));
                        *reinterpret_cast<float4*>(obase + size_t(rr) * E + c * 32 + k * 4) = f;
                    }
                    __syncwarp();
                }
                tc_fence_before_sync();  // O and the row sum are in registers before this warp's next p_full arrival
            }
            gt += uint32_t(n_t);
            go += uint32_t(n_o);
        }
        if (args.out_amax) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

df8_status launch_attention_wide(const CUtensorMap& tm, const AttnArgs& args, dim3 grid, cudaStream_t st) {
    auto kern = attention_fp8_wide_kernel;
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        DF8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WideCfg::kSmemBytes));
        configured[dev] = true;
    }
    cudaError_t err = launch_kernel(kern, grid, dim3(kWideThreads), WideCfg::kSmemBytes, st, tm, args);
    if (err != cudaSuccess) return fail(DF8_ERR_CUDA, "launch of attention_fp8_wide_kernel failed: %s", cudaGetErrorString(err));
    return DF8_OK;
}

template <int D>
df8_status launch_attention(const CUtensorMap& tm, const AttnArgs& args, dim3 grid, cudaStream_t st) {
    using Cfg = AttnCfg<D>;
    auto kern = attention_fp8_kernel<D>;
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        DF8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        configured[dev] = true;
    }
    cudaError_t err = launch_kernel(kern, grid, dim3(kAttnThreads), Cfg::kSmemBytes, st, tm, args);
    if (err != cudaSuccess) return fail(DF8_ERR_CUDA, "launch of attention_fp8_kernel failed: %s", cudaGetErrorString(err));
    return DF8_OK;
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_attention_fp8(const uint8_t* qkv_codes, df8_kind kind, const float* scale, int B, int T,
                                        int H, int D, int mask_mode, const float* mask, int mask_b, float* out,
                                        float* out_amax, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_attention_fp8: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(B >= 0 && T >= 0 && H > 0, "df8_attention_fp8: bad shape B=%d T=%d H=%d", B, T, H);
    DF8_REQUIRE(mask_mode >= 0 && mask_mode <= 2, "df8_attention_fp8: unknown mask mode %d", mask_mode);
    DF8_REQUIRE(mask_mode != 2 || (mask != nullptr && (mask_b == 1 || mask_b == B)),
                "df8_attention_fp8: additive mask must be [B,1,T,T] or [1,1,T,T]");
    if (D != 64 && D != 128)
        return fail(DF8_ERR_UNSUPPORTED, "df8_attention_fp8: head dimension %d not supported (64 or 128)", D);
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(out_amax, st);
    if (B == 0 || T == 0) return DF8_OK;
    DF8_REQUIRE(qkv_codes && scale && out, "df8_attention_fp8: null buffer");
    DF8_REQUIRE(aligned16(out), "df8_attention_fp8: out must be 16-byte aligned");
    const int E = H * D;
    const long rows = long(B) * T;
    DF8_REQUIRE(rows < (1l << 31), "df8_attention_fp8: too many tokens");

    unsigned int* status_ptr = nullptr;
    df8_status src = status_word_device_ptr(&status_ptr);
    if (src != DF8_OK) return src;

    CUtensorMap tm;
    df8_status rc = make_tmap_2d_u8(&tm, qkv_codes, uint64_t(rows), uint64_t(3 * E), uint64_t(3 * E), BQ, uint32_t(D), D);
    if (rc != DF8_OK) return rc;

    AttnArgs a;
    a.scale = scale;
    a.mask = mask;
    a.out = out;
    a.out_amax = out_amax;
    a.B = B;
    a.T = T;
    a.H = H;
    a.E = E;
    a.mask_mode = mask_mode;
    a.mask_b = mask_b;
    a.idesc_qk = ptx::make_idesc_f8(BQ, BKV, int(kind), int(kind));
    a.v_kind = int(kind);
    a.idesc_pv = ptx::make_idesc_f16(BQ, D, 0, 1);
    a.idesc_sum = ptx::make_idesc_f16(BQ, 16);
    a.status = status_ptr;
    a.n_qblk = (T + BQ - 1) / BQ;
    const long items = long(a.n_qblk) * H * B;
    DF8_REQUIRE(items < (1l << 31), "df8_attention_fp8: too many query blocks");
    a.n_items = int(items);
    // D = 64 and whole pairs of query blocks: two query tiles per CTA (DF8_ATTN_WIDE=0 in the environment keeps
    // the one-tile kernel, for profiling and tests)
    const char* wide_env = getenv("DF8_ATTN_WIDE");
    if (D == 64 && T % (2 * BQ) == 0 && !(wide_env && wide_env[0] == '0')) {
        a.idesc_pv = ptx::make_idesc_f16(BQ, WideCfg::kON, 0, 1);
        const long witems = long(T / (2 * BQ)) * H * B;
        a.n_items = int(witems);
        const long sms = sm_count();
        return launch_attention_wide(tm, a, dim3(unsigned(witems < sms ? witems : sms), 1, 1), st);
    }
    const long slots = long(sm_count()) * (D == 64 ? 2 : 1);  // CTAs resident at once
    dim3 grid(unsigned(items < slots ? items : slots), 1, 1);
    return D == 64 ? launch_attention<64>(tm, a, grid, st) : launch_attention<128>(tm, a, grid, st);
}

