// dlopen-based loader of rollout-worker plugins (RTLD_NOW | RTLD_LOCAL), requiring the two
// exported C symbols and forwarding generate / parameter queries.
// Reference: src/rollout/plugin_worker.cc:11-64.
#include "cverl/rollout_plugin.h"

#include <cstdio>
#include <dlfcn.h>
#include <string>

namespace {
struct Plugin {
  void* dl = nullptr;
  cverl_rollout_worker_t* worker = nullptr;
  cverl_destroy_rollout_worker_fn destroy = nullptr;
};
void set_err(char* err, int len, const std::string& msg) {
  if (err && len > 0) std::snprintf(err, static_cast<size_t>(len), "%s", msg.c_str());
}
}  // namespace

extern "C" {

void* cverl_plugin_load(const char* path, const char* config_json, char* err, int err_len) {
  void* dl = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!dl) {
    const char* e = dlerror();
    set_err(err, err_len, std::string("dlopen failed: ") + (e ? e : "unknown"));
    return nullptr;
  }
  auto create = reinterpret_cast<cverl_create_rollout_worker_fn>(dlsym(dl, "cverl_create_rollout_worker"));
  auto destroy = reinterpret_cast<cverl_destroy_rollout_worker_fn>(dlsym(dl, "cverl_destroy_rollout_worker"));
  if (!create || !destroy) {
    set_err(err, err_len, "plugin lacks cverl_create_rollout_worker / cverl_destroy_rollout_worker");
    dlclose(dl);
    return nullptr;
  }
  cverl_rollout_worker_t* w = create(config_json ? config_json : "{}");
  if (!w || !w->generate || !w->num_parameters || !w->parameter) {
    set_err(err, err_len, "cverl_create_rollout_worker returned no usable worker");
    if (w) destroy(w);
    dlclose(dl);
    return nullptr;
  }
  auto* p = new Plugin();
  p->dl = dl;
  p->worker = w;
  p->destroy = destroy;
  return p;
}

int cverl_plugin_generate(void* handle, const cverl_generate_args_t* args) {
  auto* p = static_cast<Plugin*>(handle);
  return p->worker->generate(p->worker->self, args);
}
int64_t cverl_plugin_num_parameters(void* handle) {
  auto* p = static_cast<Plugin*>(handle);
  return p->worker->num_parameters(p->worker->self);
}
int cverl_plugin_parameter(void* handle, int64_t index, cverl_parameter_view_t* out) {
  auto* p = static_cast<Plugin*>(handle);
  return p->worker->parameter(p->worker->self, index, out);
}
void cverl_plugin_unload(void* handle) {
  auto* p = static_cast<Plugin*>(handle);
  if (p->worker) p->destroy(p->worker);
  if (p->dl) dlclose(p->dl);
  delete p;
}
}
