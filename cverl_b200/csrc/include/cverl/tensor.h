/* Non-owning 2-D tensor views passed across the public C ABI.  Field order and
 * enum values match the reference's include/cverl/tensor.h:9-32 so that a
 * caller compiled against either header is binary compatible. */
#ifndef CVERL_TENSOR_H_
#define CVERL_TENSOR_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cverl_dtype_e { CVERL_DTYPE_F32 = 0 } cverl_dtype_t;

typedef enum cverl_device_e { CVERL_DEVICE_CPU = 0, CVERL_DEVICE_CUDA = 1 } cverl_device_t;

/* Row-major [rows, cols] view; `data` stays owned by the caller. */
typedef struct cverl_tensor2d_s {
  void* data;
  cverl_dtype_t dtype;
  cverl_device_t device;
  int64_t rows;
  int64_t cols;
} cverl_tensor2d_t;

typedef struct cverl_const_tensor2d_s {
  const void* data;
  cverl_dtype_t dtype;
  cverl_device_t device;
  int64_t rows;
  int64_t cols;
} cverl_const_tensor2d_t;

#ifdef __cplusplus
}
#endif
#endif /* CVERL_TENSOR_H_ */
