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
//   warps 2-5  epilogue:     tcgen05.ld -> smem transpose -> coalesced global stores with the fused
//                            dequant scale, bias, GELU (upstream activation_layer.cu:9-20 formula),
//                            residual add (upstream tensor.cu:383-415) and |out| max reduction
// The epilogue of tile i overlaps the main loop of tile i+1 through the second TMEM buffer.
// All mbarrier waits are bounded; a wait that gives up records a code in the status word
// (df8_status_word_read) and the CTA tears down normally.
#include "df8_internal.cuh"
#include "sm100_ptx.cuh"
#include "tensormap.cuh"

namespace df8 {

namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == fp8 elements per K-block (one 128-byte swizzle row)
constexpr int kGemmThreads = 192;
constexpr int kStagingFloatsPerWarp = 32 * 36;

struct GemmArgs {
    const float* scale_a;   // {q, dq} of A
    const float* scale_w;   // {q, dq} of W
    const float* bias;      // [N] or null
    const float* residual;  // [M,N] or null
    float* out;             // [M,N] fp32
    float* out_amax;        // 1 float or null
    int M, N, K;
    int flags;
    uint32_t idesc;
    unsigned int* status;
};

template <int BN, int STAGES>
struct GemmCfg {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagingBytes = 4 * kStagingFloatsPerWarp * 4;
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

__device__ __forceinline__ float gelu_tanh(float x) {
    // x * 0.5 * (1 + tanh(0.7978845608 * (x + 0.044715 x^3)))
    const float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
    return x * 0.5f * (1.0f + t);
}

// Epilogue for one 32-row x 32-column chunk held by one warp (thread = row, r[j] = column j).
// Transposes through the warp's staging buffer so that global accesses are coalesced along N.
template <bool VEC4>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], float* stg, int lane, int row0, int col0,
                                               const GemmArgs& a, float alpha, float& amax) {
    if constexpr (VEC4) {
        float4* srow = reinterpret_cast<float4*>(stg + lane * 36);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            srow[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        __syncwarp();
        const int cq = (lane & 7) * 4;
        const int gcol = col0 + cq;
        const bool col_ok = gcol < a.N;
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.bias && col_ok) b4 = *reinterpret_cast<const float4*>(a.bias + gcol);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int rl = it * 4 + (lane >> 3);
            const int grow = row0 + rl;
            float4 v = *reinterpret_cast<const float4*>(stg + rl * 36 + cq);
            if (grow < a.M && col_ok) {
                v.x = fmaf(v.x, alpha, b4.x);
                v.y = fmaf(v.y, alpha, b4.y);
                v.z = fmaf(v.z, alpha, b4.z);
                v.w = fmaf(v.w, alpha, b4.w);
                if (a.flags & 1) {
                    v.x = gelu_tanh(v.x);
                    v.y = gelu_tanh(v.y);
                    v.z = gelu_tanh(v.z);
                    v.w = gelu_tanh(v.w);
                }
                const size_t off = size_t(grow) * a.N + gcol;
                if (a.flags & 2) {
                    const float4 rs = *reinterpret_cast<const float4*>(a.residual + off);
                    v.x += rs.x;
                    v.y += rs.y;
                    v.z += rs.z;
                    v.w += rs.w;
                }
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                *reinterpret_cast<float4*>(a.out + off) = v;
            }
        }
        __syncwarp();
    } else {
        float* srow = stg + lane * 33;
#pragma unroll
        for (int j = 0; j < 32; ++j) srow[j] = __uint_as_float(r[j]);
        __syncwarp();
        const int gcol = col0 + lane;
        const bool col_ok = gcol < a.N;
        const float b = (a.bias && col_ok) ? a.bias[gcol] : 0.f;
#pragma unroll 8
        for (int rl = 0; rl < 32; ++rl) {
            const int grow = row0 + rl;
            float v = stg[rl * 33 + lane];
            if (grow < a.M && col_ok) {
                v = fmaf(v, alpha, b);
                if (a.flags & 1) v = gelu_tanh(v);
                const size_t off = size_t(grow) * a.N + gcol;
                if (a.flags & 2) v += a.residual[off];
                amax = fmaxf(amax, fabsf(v));
                a.out[off] = v;
            }
        }
        __syncwarp();
    }
}

template <int BN, int STAGES, bool VEC4>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_fp8_tn_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_w,
                   const GemmArgs args) {
    using Cfg = GemmCfg<BN, STAGES>;
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(tfull + b), 1);
            mbar_init(smem_u32(tempty + b), 4);
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

    const int num_m = (args.M + BM - 1) / BM;
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
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % num_m) * BM;
                const int n0 = (tile / num_m) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(empty + stage), phase ^ 1)) {
                        record_timeout(args.status, 0x100u + stage);
                        ok = false;
                        break;
                    }
                    const uint32_t fb = smem_u32(full + stage);
                    uint8_t* sa = smem + stage * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(fb, Cfg::kStageBytes);
                    tma_load_2d(smem_u32(sa), &tma_a, fb, kb * BK, m0);
                    tma_load_2d(smem_u32(sa + Cfg::kABytes), &tma_w, fb, kb * BK, n0);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
                const uint32_t buf = acc_it & 1;
                const uint32_t acc_phase = (acc_it >> 1) & 1;
                if (!mbar_wait_bounded(smem_u32(tempty + buf), acc_phase ^ 1)) {
                    record_timeout(args.status, 0x200u + buf);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(full + stage), phase)) {
                        record_timeout(args.status, 0x300u + stage);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * Cfg::kStageBytes);
                    const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        tc_mma_f8(d_tmem, make_desc_kmajor_sw128(a_addr + k * 32),
                                  make_desc_kmajor_sw128(b_addr + k * 32), args.idesc, (kb | k) != 0);
                    tc_commit(smem_u32(empty + stage));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) tc_commit(smem_u32(tfull + buf));
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        float* stg = staging + (warp - 2) * kStagingFloatsPerWarp;
        const float alpha = args.scale_a[1] * args.scale_w[1];
        uint32_t acc_it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++acc_it) {
            const uint32_t buf = acc_it & 1;
            const uint32_t acc_phase = (acc_it >> 1) & 1;
            const int m0 = (tile % num_m) * BM;
            const int n0 = (tile / num_m) * BN;
            if (!mbar_wait_bounded(smem_u32(tfull + buf), acc_phase)) {
                if (lane == 0) record_timeout(args.status, 0x400u + buf);
                break;
            }
            tc_fence_after_sync();
            float amax = 0.f;
            const int row0 = m0 + q * 32;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                if (n0 + c * 32 >= args.N) break;  // uniform across the warp
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + buf * BN + c * 32 + (uint32_t(q * 32) << 16), r);
                tmem_ld_wait();
                epilogue_chunk<VEC4>(r, stg, lane, row0, n0 + c * 32, args, alpha, amax);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tempty + buf));
            if (args.flags & 4) {
                amax = warp_max(amax);
                if (lane == 0 && amax > 0.f) atomic_max_nonneg(args.out_amax, amax);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int BN, int STAGES, bool VEC4>
df8_status launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, const GemmArgs& args, int grid,
                       cudaStream_t st) {
    using Cfg = GemmCfg<BN, STAGES>;
    auto kern = gemm_fp8_tn_kernel<BN, STAGES, VEC4>;
    static bool configured[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        DF8_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        configured[dev] = true;
    }
    kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(ta, tw, args);
    DF8_LAUNCH_CHECK("gemm_fp8_tn_kernel");
    return DF8_OK;
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_gemm_fp8_tn(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                      const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                      const float* bias, const float* residual, int M, int N, int K, int flags,
                                      float* out, float* out_amax, df8_stream stream) {
    DF8_REQUIRE((kind_a == DF8_E4M3 || kind_a == DF8_E5M2) && (kind_w == DF8_E4M3 || kind_w == DF8_E5M2),
                "df8_gemm_fp8_tn: unknown fp8 kind");
    DF8_REQUIRE(M >= 0 && N >= 0 && K > 0, "df8_gemm_fp8_tn: bad shape M=%d N=%d K=%d", M, N, K);
    DF8_REQUIRE((flags & ~7) == 0, "df8_gemm_fp8_tn: unknown flags 0x%x", flags);
    cudaStream_t st = as_stream(stream);
    if (flags & DF8_EPI_AMAX) {
        DF8_REQUIRE(out_amax != nullptr, "df8_gemm_fp8_tn: DF8_EPI_AMAX needs out_amax");
        DF8_CUDA_TRY(cudaMemsetAsync(out_amax, 0, sizeof(float), st));
    }
    if (M == 0 || N == 0) return DF8_OK;
    DF8_REQUIRE(a_codes && w_codes && scale_a && scale_w && out, "df8_gemm_fp8_tn: null buffer");
    DF8_REQUIRE(!(flags & DF8_EPI_RESIDUAL) || residual != nullptr, "df8_gemm_fp8_tn: DF8_EPI_RESIDUAL needs residual");
    if (K % 16 != 0)
        return fail(DF8_ERR_UNSUPPORTED, "df8_gemm_fp8_tn: K=%d must be a multiple of 16 (TMA row pitch)", K);

    unsigned int* status_ptr = nullptr;
    df8_status src = status_word_device_ptr(&status_ptr);
    if (src != DF8_OK) return src;

    const int sms = sm_count();
    // tile width: the one that fills whole waves of the persistent grid best (wider tiles reuse A more)
    auto efficiency = [&](int bn, double weight) {
        const long tiles = long((M + BM - 1) / BM) * ((N + bn - 1) / bn);
        const long waves = (tiles + sms - 1) / sms;
        return weight * double(tiles) / double(waves * sms) * (double(N) / double(((N + bn - 1) / bn) * bn));
    };
    const bool wide = efficiency(256, 1.0) >= efficiency(128, 0.92);
    const int bn = wide ? 256 : 128;
    const long tiles = long((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int grid = int(tiles < sms ? tiles : sms);

    CUtensorMap ta, tw;
    df8_status rc = make_tmap_2d_u8(&ta, a_codes, uint64_t(M), uint64_t(K), uint64_t(K), BM, BK, 128);
    if (rc != DF8_OK) return rc;
    rc = make_tmap_2d_u8(&tw, w_codes, uint64_t(N), uint64_t(K), uint64_t(K), uint32_t(bn), BK, 128);
    if (rc != DF8_OK) return rc;

    GemmArgs args;
    args.scale_a = scale_a;
    args.scale_w = scale_w;
    args.bias = bias;
    args.residual = residual;
    args.out = out;
    args.out_amax = out_amax;
    args.M = M;
    args.N = N;
    args.K = K;
    args.flags = flags;
    args.idesc = ptx::make_idesc_f8(BM, bn, int(kind_a), int(kind_w));
    args.status = status_ptr;

    const bool vec4 = (N % 4 == 0) && aligned16(out) && (!bias || aligned16(bias)) &&
                      (!(flags & DF8_EPI_RESIDUAL) || aligned16(residual));
    if (wide)
        return vec4 ? launch_gemm<256, 4, true>(ta, tw, args, grid, st)
                    : launch_gemm<256, 4, false>(ta, tw, args, grid, st);
    return vec4 ? launch_gemm<128, 6, true>(ta, tw, args, grid, st)
                : launch_gemm<128, 6, false>(ta, tw, args, grid, st);
}
