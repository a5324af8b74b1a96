// Public C entry points and shared host helpers of the tcgen05 GEMM family.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tnnb {

// Epilogue flags (bit-or).
enum GemmEpilogue : int {
  EPI_BIAS = 1,      // + bias[n] (bf16)
  EPI_GELU = 2,      // tanh-GELU; the pre-activation is also written to aux_out when given
  EPI_DGELU = 4,     // * gelu'(aux_in[m,n])
  EPI_RESID = 8,     // + resid[m,n] (bf16)
  EPI_RELU = 16,     // max(.,0)
  EPI_ATOMIC = 32,   // D is fp32 and receives red.add (required for split-K)
  EPI_OUT_F32 = 64,  // D is fp32 (plain store)
  EPI_ACCUM = 128,   // D += result (non-atomic read-modify-write)
};

// Encode a 128B-swizzled bf16 tiled tensor map. dims/box are innermost first;
// strides_bytes has rank-1 entries (stride of dims 1..rank-1).
int encode_tmap_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box,
                     const uint32_t* elem_strides);
int encode_tmap_f32(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box);
int sm_count();

}  // namespace tnnb

extern "C" {
// D[M,N] = op(A) * op(B)^T with a fused epilogue. a_mn/b_mn: 0 = operand
// stored [rows, K] (K contiguous), 1 = stored [K, rows]. Leading dimensions
// are in elements. Returns 0 on success, a negative code on a rejected call.
// *status (device int, may be null) receives a KernelStatus code if a bounded
// wait inside the kernel expires.
int tnnb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn,
                   long long lda, long long ldb, long long ldd, const void* bias,
                   const void* aux_in, void* aux_out, long long ld_aux, const void* resid,
                   long long ld_res, int flags, int split_k, int force_bn, int* status,
                   void* stream);
}

extern "C" {
// Tensor-parallel GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter); see gemm_tcgen05.cu and tp_flags.cuh.
int tnnb_gemm_tp(int mode, const void* A, const void* B, void* D, int M, int N, int K, int b_mn, long long lda,
                 long long ldb, long long ldd, const void* bias, const void* aux_in, void* aux_out, long long ld_aux,
                 int flags, int tp, int rank, int rows_per_rank, const void* pass, const void* a_ready, void** out,
                 long long ldo, void** arrived, int n_push, void** push_dst, void** push_ready, int push_first_block, int force_bn, int* status,
                 void* stream);
}
