/* Opaque handle type and the compute-mode enumeration of the cuMpSGEMM API.
 *
 * Drop-in counterpart of the reference's include/cumpsgemm/detail/common.h:1-21.
 * The numeric values are part of the binary contract: rule libraries and the
 * Python control module pass them as plain integers, and the device-resident
 * dynamic-launch flag word stores the mode in its low five bits.
 */
#ifndef CUMPSGEMM_B200_DETAIL_COMMON_H
#define CUMPSGEMM_B200_DETAIL_COMMON_H

struct cuMpSGEMM_handle;
typedef struct cuMpSGEMM_handle *cuMpSGEMM_handle_t;

enum cuMpSGEMM_compute_mode_t {
  CUMPSGEMM_CUBLAS = 0,           /* forward to the real cuBLAS, its own default math */
  CUMPSGEMM_FP16TCEC = 1,         /* FP16 tensor cores + error correction */
  CUMPSGEMM_TF32TCEC = 2,         /* TF32 tensor cores + error correction */
  CUMPSGEMM_FP16TC = 3,           /* FP16 tensor cores, no correction (debug) */
  CUMPSGEMM_TF32TC = 4,           /* TF32 tensor cores, no correction (debug) */
  CUMPSGEMM_CUBLAS_SIMT = 5,      /* forward to cuBLAS, FP32 SIMT */
  CUMPSGEMM_CUBLAS_FP16TC = 6,    /* forward to cuBLAS, fast FP16 */
  CUMPSGEMM_CUBLAS_TF32TC = 7,    /* forward to cuBLAS, fast TF32 */
  CUMPSGEMM_DRY_RUN = 8,          /* log only, compute nothing */
  CUMPSGEMM_AUTO = 9,             /* exponent statistics pick FP16TCEC / scaling / TF32TCEC */
  CUMPSGEMM_UNDEFINED = 10,       /* internal: statistics not decided yet */
  CUMPSGEMM_FP16TCEC_SCALING = 11,/* FP16TCEC with power-of-two pre-scaling */
  CUMPSGEMM_FP32_SIMT = 12        /* reserved, rejected */
};

#endif
