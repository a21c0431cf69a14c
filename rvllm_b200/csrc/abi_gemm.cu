// C-ABI entry points of the FP8 GEMM family: validation, kernel choice, launches.
#include <limits.h>
#include <math.h>

#include "../../include/rvllm_b200.h"
#include "../../include/rvllm_b200_tuning.h"
#include "host_util.h"
#include "fp8_gemm_stream.cuh"
#include "fp8_gemm_tc.cuh"
#include "fp8_layer_block.cuh"

extern "C" {
// ---------------------------------------------------------------- stage 2: GEMM
}  // extern "C"

namespace {

struct GemmArgs {
    void* out;
    int out_kind;
    const void* a;
    const void* w;
    const float* a_scale;
    const float* w_scale;
    const void* residual;
    int M, N, K;
};

int validate_gemm(const GemmArgs& g) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return rv_fail(RVLLM_E_INVALID, "M, N, K must be > 0");
    if (!g.out || !g.a || !g.w || !g.a_scale || !g.w_scale) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (g.out_kind < 0 || g.out_kind > 2) return rv_fail(RVLLM_E_INVALID, "unknown output kind");
    if (g.residual && g.out_kind == RVLLM_OUT_F32) return rv_fail(RVLLM_E_INVALID, "residual needs a 16-bit output");
    if ((long long)g.M * g.N > (1LL << 40) || (long long)g.N * g.K > (1LL << 42))
        return rv_fail(RVLLM_E_INVALID, "problem size overflows");
    if (g.K % 64 != 0) return rv_fail(RVLLM_E_UNSUPPORTED, "K must be a multiple of 64");
    if (!rv_aligned(g.a, 16) || !rv_aligned(g.w, 16)) return rv_fail(RVLLM_E_INVALID, "A / W must be 16-byte aligned");
    return RVLLM_OK;
}

template <int NT8, int EPI, typename OutT>
int launch_stream_one(const rvgemm::StreamParams& p, int splits, int mblocks, cudaStream_t s) {
    auto kern = rvgemm::fp8_gemm_stream_kernel<NT8, EPI, OutT>;
    const size_t smem = (size_t)rvgemm::K_WARPS * NT8 * 8 * rvgemm::TILE_N * sizeof(float);
    static RvDeviceOnce smem_once;  // per kernel instantiation and device; set once so graph capture sees launches only
    if (smem > 48 * 1024 && rv_allow_smem(smem_once, kern, (int)smem))
        return rv_fail(RVLLM_E_LAUNCH, "cannot raise dynamic shared memory for the streaming GEMM");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + rvgemm::TILE_N - 1) / rvgemm::TILE_N, splits, mblocks);
    cfg.blockDim = dim3(rvgemm::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (rv_pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return rv_fail(RVLLM_E_LAUNCH, "streaming GEMM launch: %s", cudaGetErrorString(e));
    }
    return RVLLM_OK;
}

template <int NT8>
int launch_stream_epi(const GemmArgs& g, const rvgemm::StreamParams& p, int splits, int mblocks, cudaStream_t s) {
    using namespace rvgemm;
    if (g.out_kind == RVLLM_OUT_F32) return launch_stream_one<NT8, EPI_F32, __half>(p, splits, mblocks, s);
    if (g.out_kind == RVLLM_OUT_F16)
        return g.residual ? launch_stream_one<NT8, EPI_RESIDUAL, __half>(p, splits, mblocks, s)
                          : launch_stream_one<NT8, EPI_SCALE, __half>(p, splits, mblocks, s);
    return g.residual ? launch_stream_one<NT8, EPI_RESIDUAL, __nv_bfloat16>(p, splits, mblocks, s)
                      : launch_stream_one<NT8, EPI_SCALE, __nv_bfloat16>(p, splits, mblocks, s);
}

// Split-K factor for the streaming kernel: enough CTAs for two per SM, at most the
// portable cluster size, and at least two 64-byte chunks per k-warp.
int stream_splits(int M, int N, int K, int mblocks) {
    (void)M;
    const int tiles = ((N + rvgemm::TILE_N - 1) / rvgemm::TILE_N) * mblocks;
    int s = (2 * 148 + tiles - 1) / tiles;
    const int chunks = K / rvgemm::CHUNK;
    while (s > 1 && chunks / (s * rvgemm::K_WARPS) < 2) s--;
    if (s < 1) s = 1;
    if (s > 8) s = 8;
    return s;
}

int launch_stream(const GemmArgs& g, cudaStream_t s) {
    rvgemm::StreamParams p;
    p.a = (const uint8_t*)g.a;
    p.w = (const uint8_t*)g.w;
    p.a_scale = g.a_scale;
    p.w_scale = g.w_scale;
    p.out = g.out;
    p.residual = g.residual;
    p.M = g.M;
    p.N = g.N;
    p.K = g.K;
    p.ldo = g.N;
    int nt8 = (g.M + 7) / 8;
    if (nt8 > 8) nt8 = 8;
    if (nt8 == 3) nt8 = 4;
    if (nt8 > 4 && nt8 < 8) nt8 = 8;
    const int mblocks = (g.M + nt8 * 8 - 1) / (nt8 * 8);
    const int splits = stream_splits(g.M, g.N, g.K, mblocks);
    switch (nt8) {
        case 1: return launch_stream_epi<1>(g, p, splits, mblocks, s);
        case 2: return launch_stream_epi<2>(g, p, splits, mblocks, s);
        case 4: return launch_stream_epi<4>(g, p, splits, mblocks, s);
        default: return launch_stream_epi<8>(g, p, splits, mblocks, s);
    }
}

int run_gemm(const GemmArgs& g, int impl, void* workspace, size_t workspace_size, cudaStream_t s) {
    int rc = validate_gemm(g);
    if (rc) return rc;
    if (impl == 0) impl = rvtc::prefer_tc(g.M, g.N, g.K) ? 2 : 1;
    if (impl == 2) {
        rvtc::TcArgs t;
        t.out = g.out;
        t.out_kind = g.out_kind;
        t.a = g.a;
        t.w = g.w;
        t.a_scale = g.a_scale;
        t.w_scale = g.w_scale;
        t.residual = g.residual;
        t.M = g.M;
        t.N = g.N;
        t.K = g.K;
        return rvtc::launch(t, workspace, workspace_size, s);
    }
    if (impl != 1) return rv_fail(RVLLM_E_INVALID, "impl must be 0, 1 or 2");
    return launch_stream(g, s);
}

// Device-side broadcast of a scalar weight scale is done by pointing w_scale at a
// per-channel vector; the reference's scalar-B-scale entry points are served by
// expanding the scalar into the head of the caller's workspace.
__global__ void fill_scale_kernel(float* dst, const float* scalar, int n) {
    const float v = *scalar;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = v;
}

}  // namespace

extern "C" {

size_t rvllm_fp8_gemm_workspace(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return rvtc::workspace_bytes(M, N, K);
}

int rvllm_fp8_gemm_channelscale(void* out, int out_kind, const void* a_fp8, const void* w_fp8,
                                const float* a_scale, const float* w_scale, const void* residual, int M, int N,
                                int K, int impl, void* workspace, size_t workspace_size, void* stream) {
    GemmArgs g = {out, out_kind, a_fp8, w_fp8, a_scale, w_scale, residual, M, N, K};
    return run_gemm(g, impl, workspace, workspace_size, (cudaStream_t)stream);
}

int cutlass_fp8_gemm_channelscale(void* out_f16, const void* a_fp8, const void* b_fp8, const void* row_scale,
                                  const void* col_scale, int M, int N, int K, void* workspace,
                                  size_t workspace_size, void* stream) {
    GemmArgs g = {out_f16, RVLLM_OUT_F16, a_fp8, b_fp8, (const float*)row_scale, (const float*)col_scale,
                  nullptr, M, N, K};
    return run_gemm(g, 0, workspace, workspace_size, (cudaStream_t)stream) == RVLLM_OK ? 0 : -1;
}
size_t cutlass_fp8_gemm_channelscale_workspace(int M, int N, int K) { return rvllm_fp8_gemm_workspace(M, N, K); }

static int scalar_b_gemm(void* out_f16, const void* a_fp8, const void* b_fp8, const void* a_scales,
                         const void* b_scale, const void* residual, int M, int N, int K, void* workspace,
                         size_t workspace_size, void* stream) {
    if (N <= 0 || !b_scale) return rv_fail(RVLLM_E_INVALID, "bad scalar-scale GEMM arguments");
    const size_t head = ((size_t)N * sizeof(float) + 255) & ~(size_t)255;
    if (!workspace || !rv_aligned(workspace, 16) || workspace_size < head)
        return rv_fail(RVLLM_E_WORKSPACE, "workspace too small for the expanded weight scale");
    cudaStream_t s = (cudaStream_t)stream;
    fill_scale_kernel<<<(N + 255) / 256, 256, 0, s>>>((float*)workspace, (const float*)b_scale, N);
    int rc = rv_launched("fill_scale");
    if (rc) return rc;
    GemmArgs g = {out_f16, RVLLM_OUT_F16, a_fp8, b_fp8, (const float*)a_scales, (const float*)workspace,
                  residual, M, N, K};
    return run_gemm(g, 0, (char*)workspace + head, workspace_size - head, s);
}

int cutlass_fp8_gemm_v0(void* out_f16, const void* a_fp8, const void* b_fp8, const void* a_scales,
                        const void* b_scale, int M, int N, int K, void* workspace, size_t workspace_size,
                        void* stream) {
    return scalar_b_gemm(out_f16, a_fp8, b_fp8, a_scales, b_scale, nullptr, M, N, K, workspace, workspace_size,
                         stream) == RVLLM_OK ? 0 : -1;
}
size_t cutlass_fp8_gemm_v0_workspace_size(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return (((size_t)N * sizeof(float) + 255) & ~(size_t)255) + rvllm_fp8_gemm_workspace(M, N, K);
}
int cutlass_fp8_gemm_residual_v0(void* out_f16, const void* a_fp8, const void* b_fp8, const void* a_scales,
                                 const void* b_scale, const void* residual_f16, int M, int N, int K,
                                 void* workspace, size_t workspace_size, void* stream) {
    if (!residual_f16) return -1;
    return scalar_b_gemm(out_f16, a_fp8, b_fp8, a_scales, b_scale, residual_f16, M, N, K, workspace,
                         workspace_size, stream) == RVLLM_OK ? 0 : -1;
}
size_t cutlass_fp8_gemm_residual_v0_workspace_size(int M, int N, int K) {
    return cutlass_fp8_gemm_v0_workspace_size(M, N, K);
}

int rvllm_fp8_gemm_tc_status(int* status, int reset) {
    if (!status) return rv_fail(RVLLM_E_INVALID, "status pointer is null");
    return rvtc::read_status(status, reset != 0) == 0 ? RVLLM_OK : rv_fail(RVLLM_E_LAUNCH, "cannot read the status word");
}

void rvllm_fp8_gemm_tc_tune(int stages, int splits) {
    rvtc::tune().stages = stages;
    rvtc::tune().splits = splits;
}

int rvllm_fp8_gemm_qkv_rope_fp8kv(const void* a_fp8, const void* w_fp8, const float* a_scale, const float* w_scale, int M,
                                  int K, int heads, int kv_heads, int head_dim, int dtype, void* q_fp8, float* q_scale,
                                  void* k_cache, void* v_cache, float* k_scale_cache, float* v_scale_cache,
                                  const void* cos_table, const void* sin_table, const int32_t* positions,
                                  const int32_t* slot_mapping, int max_positions, int num_cache_slots, void* stream) {
    if (head_dim != 128) return rv_fail(RVLLM_E_UNSUPPORTED, "fused QKV epilogue: head_dim must be 128 (one weight tile per head)");
    if (M <= 0 || K <= 0 || heads <= 0 || kv_heads <= 0 || max_positions <= 0 || num_cache_slots <= 0)
        return rv_fail(RVLLM_E_INVALID, "M, K, heads, kv_heads, max_positions, num_cache_slots must be > 0");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    if (!a_fp8 || !w_fp8 || !a_scale || !w_scale || !q_fp8 || !q_scale || !k_cache || !v_cache || !k_scale_cache ||
        !v_scale_cache || !cos_table || !sin_table || !positions || !slot_mapping)
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (!rv_aligned(a_fp8, 16) || !rv_aligned(w_fp8, 16)) return rv_fail(RVLLM_E_INVALID, "a / w must be 16-byte aligned");
    rvtc::TcArgs t = {};
    t.out = nullptr;
    t.out_kind = dtype;
    t.a = a_fp8;
    t.w = w_fp8;
    t.a_scale = a_scale;
    t.w_scale = w_scale;
    t.residual = nullptr;
    t.M = M;
    t.N = (heads + 2 * kv_heads) * 128;
    t.K = K;
    rvtc::RopeKv rk = {(uint8_t*)q_fp8, q_scale, (uint8_t*)k_cache, (uint8_t*)v_cache, k_scale_cache, v_scale_cache,
                       cos_table, sin_table, positions, slot_mapping, heads, kv_heads, max_positions, num_cache_slots};
    const int rc = rvtc::launch_qkv_rope(t, rk, dtype == RVLLM_F16 ? 0 : 1, (cudaStream_t)stream);
    if (rc == -3) return RVLLM_E_UNSUPPORTED;  // message already recorded
    return rc;
}

int rvllm_fp8_gemm_residual_from16(void* out, int dtype, const void* a16, const float* amax_partials, int amax_parts,
                                   const void* w_fp8, const float* w_scale, const void* residual, int M, int N, int K,
                                   void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || amax_parts <= 0) return rv_fail(RVLLM_E_INVALID, "M, N, K, amax_parts must be > 0");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    if (!out || !a16 || !amax_partials || !w_fp8 || !w_scale || !residual) return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (!rv_aligned(a16, 16) || !rv_aligned(w_fp8, 16)) return rv_fail(RVLLM_E_INVALID, "a16 / w must be 16-byte aligned");
    rvtc::TcArgs t = {};
    t.out = out;
    t.out_kind = dtype;
    t.a = nullptr;
    t.w = w_fp8;
    t.a_scale = nullptr;
    t.w_scale = w_scale;
    t.residual = residual;
    t.M = M;
    t.N = N;
    t.K = K;
    t.a16 = a16;
    t.amax_part = amax_partials;
    t.amax_parts = amax_parts;
    const int rc = rvtc::launch_residual_a16(t, dtype == RVLLM_F16 ? 0 : 1, (cudaStream_t)stream);
    if (rc == -3) return RVLLM_E_UNSUPPORTED;
    return rc;
}

int rvllm_fp8_gemm_tc_trace(void* device_u64_buffer, int slots) {
    rvtc::tune().trace = slots > 0 ? reinterpret_cast<unsigned long long*>(device_u64_buffer) : nullptr;
    rvtc::tune().trace_slots = slots > 0 ? slots : 0;
    rvtc::tune().trace_next = 0;
#if RVLLM_TC_TRACE
    return RVLLM_OK;
#else
    return device_u64_buffer && slots > 0
               ? rv_fail(RVLLM_E_UNSUPPORTED, "the GEMM time stamps are not compiled into this build (RVLLM_TC_TRACE=1 python -m rvllm_b200.build)")
               : RVLLM_OK;
#endif
}
void rvllm_fp8_gemm_tc_split_for(int slot, int N, int K, int splits) {
    if (slot < 0 || slot >= 4) return;
    rvtc::tune().split_for[slot] = (splits >= 1 && splits <= 8 && N > 0 && K > 0)
                                       ? (((long long)N << 40) | ((long long)K << 8) | (long long)splits) : 0ll;
}
void rvllm_fp8_gemm_tc_split_target(int ctas) { rvtc::tune().split_target = ctas > 0 ? ctas : 0; }
void rvllm_fp8_gemm_tc_reduce(int mode) { rvtc::tune().reduce = mode >= 1 && mode <= 3 ? mode : 0; }

size_t rvllm_fp8_gemm_gateup_workspace(int M, int I, int K) {
    if (M <= 0 || I <= 0 || K <= 0) return 0;
    const size_t stage = ((size_t)M * 2 * (size_t)I * 2 + 255) & ~(size_t)255;
    return stage + rvllm_fp8_gemm_workspace(M, 2 * I, K);
}

int rvllm_fp8_gemm_gateup_act_quant(void* out_fp8, float* out_scale, const void* a_fp8, const void* w_fp8,
                                    const float* a_scale, const float* w_scale, int M, int I, int K, int act,
                                    int dtype, int impl, void* workspace, size_t workspace_size, void* stream) {
    if (M <= 0 || I <= 0 || K <= 0 || I > INT_MAX / 2) return rv_fail(RVLLM_E_INVALID, "M, I, K must be > 0");
    int rc = rvllm_fused_act_mul_fp8_quant_validate((uint32_t)M, (uint32_t)I);
    if (rc) return rc;
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    if (act != RVLLM_ACT_SILU && act != RVLLM_ACT_GELU_TANH) return rv_fail(RVLLM_E_INVALID, "unknown activation");
    if (impl < 0 || impl > 3) return rv_fail(RVLLM_E_INVALID, "impl must be 0..3");
    const size_t stage = ((size_t)M * 2 * (size_t)I * 2 + 255) & ~(size_t)255;
    if (!workspace || !rv_aligned(workspace, 256) || workspace_size < rvllm_fp8_gemm_gateup_workspace(M, I, K))
        return rv_fail(RVLLM_E_WORKSPACE, "gate-up workspace missing, misaligned or too small");
    // One launch where the layer-block kernel's gate|up stage takes the shape (batch <= 32, K a multiple of 128 up to
    // 6144, I a multiple of 64 up to 4 * K): gate and up rows of the same 64 columns are one 128-row operand, the
    // epilogue rounds both to the 16-bit type, multiplies, keeps the products on chip, the grid meets once for the
    // row maxima and quantises — the [M, 2*I] intermediate never reaches HBM.  Same bytes as the two launches below.
    if (impl == 0 || impl == 3) {
        const bool takes = rvblk::blk_shape_ok(M, K, I, K) && rv_aligned(a_fp8, 16) && rv_aligned(w_fp8, 16) &&
                           rv_aligned(out_fp8, 16) && a_scale && w_scale && out_scale &&
                           workspace_size >= 256 + rvblk::blk_amax_bytes(I);
        if (takes) {
            rvblk::BlkArgs b = {};
            b.M = M;
            b.H = K;
            b.F = I;
            b.KO = K;
            b.act = act;
            b.dtype = dtype == RVLLM_F16 ? 0 : 1;
            b.phases = rvblk::PH_GU;
            b.eps = 0.0f;
            b.attn16 = a_fp8;  // (stages that are not run: any valid address, never read)
            b.o_w = w_fp8;
            b.d_w = w_fp8;
            b.x8 = const_cast<void*>(a_fp8);
            b.xs = const_cast<float*>(a_scale);
            b.gu_w = w_fp8;
            b.gu_wscale = w_scale;
            b.h8 = out_fp8;
            b.hs = out_scale;
            b.workspace = workspace;
            b.workspace_bytes = workspace_size;
            // the grid barrier's words: zero before a launch (every launch leaves them zero, but the two-launch form
            // of this call uses the same bytes as its staging buffer)
            if (cudaMemsetAsync(workspace, 0, 256, (cudaStream_t)stream) != cudaSuccess) {
                cudaGetLastError();
                return rv_fail(RVLLM_E_LAUNCH, "cannot clear the gate-up barrier words");
            }
            rc = rvblk::launch_block(b, (cudaStream_t)stream);
            if (rc == 0) return RVLLM_OK;
            if (rc != -3) return rc;
        }
        if (impl == 3) return rv_fail(RVLLM_E_UNSUPPORTED, "gate-up single launch: shape not taken");
    }
    // Two launches.  The projection lands in the 16-bit type the standalone chain would use, so the
    // activation + re-quantisation sees bit-identical inputs either way.
    GemmArgs g = {workspace, dtype == RVLLM_F16 ? RVLLM_OUT_F16 : RVLLM_OUT_BF16, a_fp8, w_fp8, a_scale, w_scale,
                  nullptr, M, 2 * I, K};
    rc = run_gemm(g, impl == 3 ? 0 : impl, (char*)workspace + stage, workspace_size - stage, (cudaStream_t)stream);
    if (rc) return rc;
    return rvllm_fused_act_mul_fp8_quant_launch((uint32_t)M, (uint32_t)I, act, out_fp8, out_scale, workspace, dtype,
                                                stream);
}

size_t rvllm_fp8_gemm_lm_head_argmax_workspace(int M, int vocab) {
    if (M <= 0 || vocab <= 0) return 0;
    const size_t tiles = ((size_t)vocab + 127) / 128;
    return 2 * (((size_t)M * tiles * 4 + 255) & ~(size_t)255);
}

int rvllm_fp8_gemm_lm_head_argmax(int32_t* out_tokens, const void* a_fp8, const void* w_fp8, const float* a_scale,
                                  const float* w_scale, int M, int vocab, int K, float softcap, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    GemmArgs g = {out_tokens, RVLLM_OUT_F32, a_fp8, w_fp8, a_scale, w_scale, nullptr, M, vocab, K};
    int rc = validate_gemm(g);
    if (rc) return rc;
    if (!isfinite(softcap) || softcap < 0.0f) return rv_fail(RVLLM_E_INVALID, "softcap must be finite and >= 0 (0 = none)");
    if (K % 16 != 0) return rv_fail(RVLLM_E_UNSUPPORTED, "K must be a multiple of 16");
    const size_t need = rvllm_fp8_gemm_lm_head_argmax_workspace(M, vocab);
    if (!workspace || !rv_aligned(workspace, 256) || workspace_bytes < need)
        return rv_fail(RVLLM_E_WORKSPACE, "argmax workspace missing, misaligned or too small");
    rvtc::TcArgs t;
    t.out = nullptr;
    t.out_kind = RVLLM_OUT_F32;
    t.a = a_fp8;
    t.w = w_fp8;
    t.a_scale = a_scale;
    t.w_scale = w_scale;
    t.residual = nullptr;
    t.M = M;
    t.N = vocab;
    t.K = K;
    t.arg_val = (float*)workspace;
    t.arg_idx = (int*)((char*)workspace + need / 2);
    t.softcap = softcap;
    rc = rvtc::launch_argmax(t, out_tokens, (cudaStream_t)stream);
    if (rc == -3) return RVLLM_E_UNSUPPORTED;
    return rc;
}

void rvllm_fp8_layer_block_trace(void* device_u64_buffer) {
    rvblk::trace_buffer().store((unsigned long long*)device_u64_buffer);
}

int rvllm_fp8_layer_block_capacity(int* ctas_per_sm, int* sms, int carveout_percent) {
    if (!ctas_per_sm || !sms) return rv_fail(RVLLM_E_INVALID, "null argument");
    return rvblk::block_capacity(ctas_per_sm, sms, carveout_percent) == 0 ? RVLLM_OK : rv_fail(RVLLM_E_LAUNCH, "occupancy query failed");
}

size_t rvllm_fp8_layer_block_workspace(int hidden, int ffn) {
    if (ffn <= 0 || ffn % 64 != 0 || hidden <= 0 || hidden % 128 != 0) return 0;
    return rvblk::blk_workspace_bytes(ffn, hidden);
}

int rvllm_fp8_layer_block(int M, int hidden, int ffn, int o_k, int act, int dtype, float eps, const void* attn_out16,
                          const float* attn_amax, int amax_parts, const void* attn_fp8, const float* attn_scale,
                          const void* o_w, const float* o_scale, void* residual, const void* mlp_norm_gamma,
                          const void* next_norm_gamma, void* x_fp8, float* x_scale, const void* gateup_w,
                          const float* gateup_scale, void* h_fp8, float* h_scale, const void* down_w,
                          const float* down_scale, void* workspace, size_t workspace_bytes, int stages, void* stream) {
    if (M <= 0 || hidden <= 0 || ffn <= 0 || o_k <= 0) return rv_fail(RVLLM_E_INVALID, "M, hidden, ffn, o_k must be > 0");
    if (dtype != RVLLM_F16 && dtype != RVLLM_BF16) return rv_fail(RVLLM_E_INVALID, "dtype must be f16 or bf16");
    if (act != RVLLM_ACT_SILU && act != RVLLM_ACT_GELU_TANH) return rv_fail(RVLLM_E_INVALID, "unknown activation");
    if (!isfinite(eps) || eps < 0.0f) return rv_fail(RVLLM_E_INVALID, "eps must be finite and >= 0");
    if (stages <= 0 || stages > 31) return rv_fail(RVLLM_E_INVALID, "stages must be a non-empty mask of RVLLM_BLOCK_*");
    if (!rvblk::blk_shape_ok(M, hidden, ffn, o_k))
        return rv_fail(RVLLM_E_UNSUPPORTED, "layer block: shape not taken (M <= 32, hidden %% 128 == 0 and <= 6144, "
                                            "ffn %% 64 == 0 and <= 4 * hidden)");
    const bool o = stages & rvblk::PH_O, n1 = stages & rvblk::PH_N1, gu = stages & rvblk::PH_GU, d = stages & rvblk::PH_D,
               n2 = stages & rvblk::PH_N2;
    if (o && !((attn_out16 && attn_amax && amax_parts > 0) || (attn_fp8 && attn_scale)))
        return rv_fail(RVLLM_E_INVALID, "O stage: give the attention output as 16-bit values + partial maxima or as FP8 rows + scales");
    if ((o && (!o_w || !o_scale)) || ((o || d || n1 || n2) && !residual) || (n1 && !mlp_norm_gamma) ||
        ((n1 || gu || n2) && (!x_fp8 || !x_scale)) || (gu && (!gateup_w || !gateup_scale)) ||
        ((gu || d) && (!h_fp8 || !h_scale)) || (d && (!down_w || !down_scale)) || !o_w || !gateup_w || !down_w || !x_fp8 || !h_fp8)
        return rv_fail(RVLLM_E_INVALID, "null device pointer");
    if (!rv_aligned(o_w, 16) || !rv_aligned(gateup_w, 16) || !rv_aligned(down_w, 16) || !rv_aligned(x_fp8, 16) ||
        !rv_aligned(h_fp8, 16) || (attn_out16 && !rv_aligned(attn_out16, 16)) || (attn_fp8 && !rv_aligned(attn_fp8, 16)) ||
        (residual && !rv_aligned(residual, 16)))
        return rv_fail(RVLLM_E_INVALID, "operands must be 16-byte aligned");
    if ((o_scale && !rv_aligned(o_scale, 16)) || (down_scale && !rv_aligned(down_scale, 16)) ||
        (mlp_norm_gamma && !rv_aligned(mlp_norm_gamma, 16)) || (next_norm_gamma && !rv_aligned(next_norm_gamma, 16)))
        return rv_fail(RVLLM_E_INVALID, "weight scales and norm gains must be 16-byte aligned");
    if (!workspace || !rv_aligned(workspace, 256) || workspace_bytes < rvblk::blk_workspace_bytes(ffn, hidden))
        return rv_fail(RVLLM_E_WORKSPACE, "layer-block workspace missing, misaligned or too small");
    rvblk::BlkArgs g = {};
    g.M = M;
    g.H = hidden;
    g.F = ffn;
    g.KO = o_k;
    g.act = act;
    g.dtype = dtype == RVLLM_F16 ? 0 : 1;
    g.phases = stages;
    g.eps = eps;
    g.attn16 = attn_out16;
    g.attn_amax = attn_amax;
    g.amax_parts = amax_parts;
    g.attn_fp8 = attn_out16 ? nullptr : attn_fp8;
    g.attn_scale = attn_scale;
    g.o_w = o_w;
    g.o_wscale = o_scale;
    g.residual = residual;
    g.gamma1 = mlp_norm_gamma;
    g.gamma2 = next_norm_gamma;
    g.x8 = x_fp8;
    g.xs = x_scale;
    g.gu_w = gateup_w;
    g.gu_wscale = gateup_scale;
    g.h8 = h_fp8;
    g.hs = h_scale;
    g.d_w = down_w;
    g.d_wscale = down_scale;
    g.workspace = workspace;
    g.workspace_bytes = workspace_bytes;
    const int rc = rvblk::launch_block(g, (cudaStream_t)stream);
    if (rc == -3) return RVLLM_E_UNSUPPORTED;
    return rc;
}

}  // extern "C"
