/* TEST INFRASTRUCTURE ONLY.
 *
 * One module image for the reference's unmodified GPU trainer (model/gpu_train.c looks up 26 kernels by name in a
 * single module, :156-180): the reference's own non-GEMM kernels, compiled here from cuda/train_kernels.cu where
 * it lies in the reference checkout (-I<reference root>), with its nine GEMM entry points renamed out of the way,
 * plus this library's GEMM entries under the reference's names.  Loading this image instead of the reference's
 * cubin swaps exactly the GEMM kernels and nothing else, which is what the drop-in test and timing need.
 */
#define k_gemm_nn ref_k_gemm_nn
#define k_gemm_nt ref_k_gemm_nt
#define k_gemm_tn ref_k_gemm_tn
#define k_bf16_gemm_nn ref_k_bf16_gemm_nn
#define k_bf16_gemm_nt ref_k_bf16_gemm_nt
#define k_bf16_gemm_tn ref_k_bf16_gemm_tn
#define k_bf16_gemm_tn_small ref_k_bf16_gemm_tn_small
#define k_bf16_gemm_nn_bias ref_k_bf16_gemm_nn_bias
#include "cuda/train_kernels.cu"
#undef k_gemm_nn
#undef k_gemm_nt
#undef k_gemm_tn
#undef k_bf16_gemm_nn
#undef k_bf16_gemm_nt
#undef k_bf16_gemm_tn
#undef k_bf16_gemm_tn_small
#undef k_bf16_gemm_nn_bias
#include "gemm_ref_abi.cu"
