/*
 * slinoss_b200 self-test library (libslinoss_b200_selftest.so): entry points that
 * exist for the test-suite only and are not part of the shipped library.
 */
#ifndef SLINOSS_B200_SELFTEST_H_
#define SLINOSS_B200_SELFTEST_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Self-test of the tcgen05 tile engine (no counterpart in the reference): one
 * CTA computes a small bf16 product with fp32 accumulation in tensor memory.
 * mode 0: C[128x128] = A[128x64] B[128x64]^T;  mode 1: C[128x64] = A[128x128]
 * B[128x64];  mode 2: C[128x64] = A[128x128]^T B[128x64];  mode 3: C[128x64] =
 * A[128x64] B[64x64]^T.  A, B row-major bf16; *status (device int) becomes 1 if
 * a bounded wait ran out.  Returns 0, a negative argument error or a positive
 * cudaError_t like the main library. */
int slx_umma_selftest(int mode, const void *A, const void *B, float *C,
                      int *status, void *stream);
const char *slx_selftest_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* SLINOSS_B200_SELFTEST_H_ */
