/* C ABI of rollout-worker plugins.
 *
 * A plugin is a shared object that exports the two symbols the reference's loader looks
 * up (include/cverl/rollout/plugin_worker.h:16-20):
 *
 *     cverl_rollout_worker_t* cverl_create_rollout_worker(const char* config_json);
 *     void cverl_destroy_rollout_worker(cverl_rollout_worker_t* worker);
 *
 * The reference hands a C++ object with virtual functions across that boundary; here the
 * worker is a plain C struct of function pointers, so a plugin needs no C++ runtime
 * agreement with the host.  Tensors are row-major host (or device) buffers owned by the
 * caller for inputs and outputs, and by the plugin for parameters. */
#ifndef CVERL_ROLLOUT_PLUGIN_H_
#define CVERL_ROLLOUT_PLUGIN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cverl_generation_config_s {
  int64_t max_new_tokens;
  double temperature;
  double top_p;
  int64_t top_k;
  int64_t eos_token_id;
  int64_t eos_check_interval;
  uint64_t seed;
} cverl_generation_config_t;

typedef struct cverl_generate_args_s {
  const int64_t* token_ids;      /* [batch, prompt_len] left-padded prompts */
  const int64_t* attention_mask; /* [batch, prompt_len] */
  const int64_t* lengths;        /* [batch] */
  int64_t batch;
  int64_t prompt_len;
  cverl_generation_config_t config;
  int64_t* out_token_ids;        /* [batch, max_new_tokens] */
  float* out_logprobs;           /* [batch, max_new_tokens] */
  int64_t* out_lengths;          /* [batch] */
} cverl_generate_args_t;

typedef struct cverl_parameter_view_s {
  const char* name;
  void* data;
  int32_t dtype;   /* 0 F32, 1 F16, 2 BF16 */
  int32_t device;  /* 0 CPU, 1 CUDA */
  int32_t ndim;
  int64_t shape[8];
} cverl_parameter_view_t;

typedef struct cverl_rollout_worker_s {
  void* self;
  int (*generate)(void* self, const cverl_generate_args_t* args);                 /* 0 on success */
  int64_t (*num_parameters)(void* self);
  int (*parameter)(void* self, int64_t index, cverl_parameter_view_t* out);       /* 0 on success */
} cverl_rollout_worker_t;

typedef cverl_rollout_worker_t* (*cverl_create_rollout_worker_fn)(const char* config_json);
typedef void (*cverl_destroy_rollout_worker_fn)(cverl_rollout_worker_t* worker);

/* Host-side loader (libcverl.so). */
void* cverl_plugin_load(const char* path, const char* config_json, char* err, int err_len);
int cverl_plugin_generate(void* handle, const cverl_generate_args_t* args);
int64_t cverl_plugin_num_parameters(void* handle);
int cverl_plugin_parameter(void* handle, int64_t index, cverl_parameter_view_t* out);
void cverl_plugin_unload(void* handle);

#ifdef __cplusplus
}
#endif
#endif /* CVERL_ROLLOUT_PLUGIN_H_ */
