// Launchers that other translation units of the library call. Argument conventions are documented
// at each definition.
#pragma once

extern "C" {

int lb_colsum(const float* partial, int P, int C, void* out, int out_fp32, int accumulate,
              void* stream);

// row/norm.cu
int lb_norm_bwd_partial_rows();
int lb_rms_norm_fwd(const void* x, const void* res_in, const void* w, void* y, void* res_out,
                    float* rstd, int N, int H, float eps, float w_off, void* stream);
int lb_rms_norm_bwd(const void* dy, const void* dres, const void* xin, const void* w,
                    const float* rstd, void* dx, float* scratch, void* dw_out, int dw_fp32,
                    int dw_accumulate, int N, int H, float w_off, void* stream);

// row/rope.cu
int lb_rope_bwd_partial_rows();
int lb_qk_norm_rope_fwd(const void* q_in, long long ldq_in, const void* k_in, long long ldk_in,
                        const void* qw, const void* kw, const float* cos, const float* sin,
                        const void* pos, int pos_i64, int pos_mod, void* q_out, long long ldq_out,
                        void* k_out, long long ldk_out, float* q_rstd, float* k_rstd, int T, int Hq,
                        int Hk, int hd, float eps, float w_off, int do_norm, void* stream);
int lb_qk_norm_rope_bwd(const void* dq, long long lddq, const void* dk, long long lddk,
                        const void* q_in, long long ldq_in, const void* k_in, long long ldk_in,
                        const void* qw, const void* kw, const float* cos, const float* sin,
                        const void* pos, int pos_i64, int pos_mod, const float* q_rstd,
                        const float* k_rstd, void* dq_in, long long lddq_in, void* dk_in,
                        long long lddk_in, float* scratch, void* dw_out, int dw_fp32,
                        int dw_accumulate, int T, int Hq, int Hk, int hd, float w_off, int do_norm,
                        void* stream);

// row/act.cu
int lb_glu_fwd(int kind, const void* gate, const void* up, long long ld_in, void* out,
               long long ld_out, long long T, int I, void* stream);
int lb_glu_bwd(int kind, const void* dout, long long ld_dout, const void* gate, const void* up,
               long long ld_in, void* dgate, void* dup, long long ld_d, long long T, int I,
               void* stream);

// attn/
int lb_attn_zero_tail(const int* plan, int capacity, int T, void* p0, long long ld0, int w0,
                      void* p1, long long ld1, int w1, void* p2, long long ld2, int w2,
                      void* stream);
int lb_attn_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                long long ldv, const int* seq_start, const int* seq_end, const int* plan,
                int max_tiles, void* o, long long ldo, float* lse, int T, int Hq, int Hk, int hd,
                float softmax_scale, int causal, int* status, void* stream);
int lb_attn_bwd(const void* dO, long long lddo, const void* q, long long ldq, const void* k,
                long long ldk, const void* v, long long ldv, const void* o, long long ldo,
                const float* lse, float* delta, const int* seq_start, const int* seq_end,
                const int* plan_q, int cap_q, const int* plan_kv, int cap_kv, void* dq,
                long long lddq, void* dk, long long lddk, void* dv, long long lddv, int T, int Hq,
                int Hk, int hd, float softmax_scale, int causal, int* status, void* stream);

// gemm/gemm_bf16.cu
int lb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                 const void* bias, int splits, int bn, int* status, void* stream);
int lb_gemm_bf16_ext(const void* A, const void* B, const void* A2, const void* B2, void* C, int M,
                     int N, int K, int K2, long long lda, long long ldb, long long lda2,
                     long long ldb2, long long ldc, int b_mn, const void* bias, int* status,
                     void* stream);
int lb_gemm_bf16_scatter16(const void* A, const void* B, const void* const* c_peers, int world,
                           int rows_per_peer, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int a_mn, int b_mn, int bn, int* status, void* stream);

int lb_gemm_bf16_push16(const void* A, const void* B, const void* const* c_peers, int world,
                        int rows_per_peer, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int bn, int* status, void* stream);
int lb_gemm_bf16_ag(const void* const* a_peers, void* a_all, const void* B, void* C, int rows_local,
                    int world, int rank, int N, int K, long long lda, long long ldb, long long ldc,
                    int b_mn, const void* bias, unsigned* flags, unsigned* counter, unsigned epoch,
                    int* status, void* stream);

// comm/
int lb_device_barrier(const void* const* pads, int world, int rank, unsigned epoch,
                      unsigned long long limit_ns, int* status, void* stream);
int lb_take_clear(void* acc, void* out, long long n, int acc_fp32, void* stream);
int lb_take_sum(const void* slots, void* out, long long n, int world, void* stream);

}  // extern "C"
