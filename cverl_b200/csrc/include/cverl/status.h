/* Status codes of the public C ABI.  Numeric values are part of the ABI and
 * match the reference's include/cverl/status.h:7-13. */
#ifndef CVERL_STATUS_H_
#define CVERL_STATUS_H_

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cverl_status_e {
  CVERL_OK = 0,                   /* success */
  CVERL_ERR_INVALID_ARGUMENT = 1, /* null pointer, wrong dtype/device, shape mismatch, bad scalar */
  CVERL_ERR_UNSUPPORTED = 2       /* valid request that this build cannot serve */
} cverl_status_t;

/* Static, NUL-terminated description of a status code (never NULL). */
const char* cverl_status_string(cverl_status_t status);

#ifdef __cplusplus
}
#endif
#endif /* CVERL_STATUS_H_ */
