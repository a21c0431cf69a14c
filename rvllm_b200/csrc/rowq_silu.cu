// PTX module `fused_silu_fp8_quant`: SiLU(gate) * up + per-token FP8 quantisation.
// Entry-point contract: kernels/fused_silu_fp8_quant.cu:42 of the reference
// (out_fp8, scales, gate_up, intermediate); body in rowq_act.cuh.
#include "rowq_act.cuh"

extern "C" __global__ void __launch_bounds__(1024)
fused_silu_mul_fp8_quant_kernel(uint8_t* out, float* scales, const __half* gate_up, int intermediate) {
    rvact::act_mul_quant_row<rvact::ACT_SILU, __half>(out, scales, gate_up, intermediate);
}
extern "C" __global__ void __launch_bounds__(1024)
fused_silu_mul_fp8_quant_bf16_kernel(uint8_t* out, float* scales, const __nv_bfloat16* gate_up, int intermediate) {
    rvact::act_mul_quant_row<rvact::ACT_SILU, __nv_bfloat16>(out, scales, gate_up, intermediate);
}
