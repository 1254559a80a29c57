// extern "C" surface of libkatab200.so (include/katab200.h).  Every entry point converts
// exceptions into a status code plus a thread-local message; nothing throws across the ABI.
#include "../../include/katab200.h"

#include <cstring>
#include <memory>
#include <string>

#include "kb_engine.h"
#include "kb_tile_table.h"

struct kb_model {
  kb::Model m;
};
struct kb_handle {
  std::unique_ptr<kb::Engine> e;
};

namespace {
thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  }
  catch(const kb::CudaError& e) { g_err = e.what(); return 2; }
  catch(const std::exception& e) { g_err = e.what(); return 1; }
  catch(...) { g_err = "unknown error"; return 3; }
}
void need(const void* p, const char* what) {
  if(p == nullptr) throw std::runtime_error(std::string(what) + " is NULL");
}
}  // namespace

extern "C" {

const char* kb_last_error(void) { return g_err.c_str(); }
const char* kb_version(void) { return "katab200 0.1 (sm_100a)"; }

int kb_device_count(int* count) {
  return guarded([&]() {
    need(count, "count");
    *count = 0;
    kb::cudaCheck(cudaGetDeviceCount(count), "cudaGetDeviceCount");
  });
}

int kb_device_name(int device, char* buf, size_t buflen) {
  return guarded([&]() {
    need(buf, "buf");
    if(buflen == 0) throw std::runtime_error("buflen is 0");
    cudaDeviceProp prop;
    kb::cudaCheck(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    std::string s = std::string(prop.name) + " (compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                    ", " + std::to_string(prop.multiProcessorCount) + " SMs, " + std::to_string(prop.totalGlobalMem >> 20) + " MiB)";
    std::strncpy(buf, s.c_str(), buflen - 1);
    buf[buflen - 1] = 0;
  });
}

int kb_model_create(const void* blob, size_t nbytes, kb_model** out) {
  if(out) *out = nullptr;
  return guarded([&]() {
    need(out, "out");
    auto m = std::make_unique<kb_model>();
    kb::parseModel(blob, nbytes, m->m);
    *out = m.release();
  });
}
void kb_model_destroy(kb_model* m) { delete m; }

int kb_model_info(const kb_model* m, int32_t info[9]) {
  return guarded([&]() {
    need(m, "model"); need(info, "info");
    const kb::Model& k = m->m;
    info[0] = k.modelVersion; info[1] = k.inC; info[2] = k.inGlobalC; info[3] = k.policyC; info[4] = k.valueC;
    info[5] = k.scoreValueC; info[6] = k.ownershipC; info[7] = k.trunkC; info[8] = k.numBlocks;
  });
}

int kb_model_meta_channels(const kb_model* m, int32_t* channels) {
  return guarded([&]() { need(m, "model"); need(channels, "channels"); *channels = m->m.inMetaC; });
}

int kb_handle_create(
  const kb_model* m, int device, int maxBatch, int nnXLen, int nnYLen, int precision, int requireExactNNLen, kb_handle** out) {
  if(out) *out = nullptr;
  return guarded([&]() {
    need(m, "model"); need(out, "out");
    auto h = std::make_unique<kb_handle>();
    h->e = std::make_unique<kb::Engine>(m->m, device, maxBatch, nnXLen, nnYLen, precision, requireExactNNLen != 0);
    *out = h.release();
  });
}
void kb_handle_destroy(kb_handle* h) { delete h; }

int kb_weight_cache_stats(int64_t stats[4]) {
  return guarded([&]() {
    need(stats, "stats");
    const kb::WeightCacheStats s = kb::weightCacheStats();
    stats[0] = s.entries; stats[1] = s.bytes; stats[2] = s.uploads; stats[3] = s.hits;
  });
}

int kb_tile_plan(int k, int inC, int outC, int32_t plan[6]) {
  return guarded([&]() {
    need(plan, "plan");
    bool fromTable = false;
    const kb::TileRow r = kb::tilePlanFor(k, inC, outC, &fromTable);
    plan[0] = r.BN; plan[1] = r.pair; plan[2] = r.epiWarps; plan[3] = r.epiWarpsRes; plan[4] = r.chain; plan[5] = fromTable ? 1 : 0;
  });
}
int kb_tile_table(int32_t* rows, int cap, int32_t* count) {
  return guarded([&]() {
    need(count, "count");
    const int n = (int)(sizeof(kb::TILE_TABLE) / sizeof(kb::TILE_TABLE[0]));
    *count = n;
    for(int i = 0; i < n && i < cap && rows; i++) {
      const kb::TileRow& r = kb::TILE_TABLE[i];
      const int32_t v[8] = {r.k, r.inC, r.outC, r.BN, r.pair, r.epiWarps, r.epiWarpsRes, r.chain};
      for(int j = 0; j < 8; j++) rows[i * 8 + j] = v[j];
    }
  });
}

int kb_selftest_wait_timeout(kb_handle* h, unsigned long long limitNs) {
  return guarded([&]() { need(h, "handle"); h->e->selfTestWaitTimeout(limitNs); });
}

int kb_handle_precision(const kb_handle* h, int* precision) {
  return guarded([&]() { need(h, "handle"); need(precision, "precision"); *precision = h->e->precision(); });
}

int kb_upload_inputs(kb_handle* h, int n, const float* spatial, const float* global, const int32_t* symmetry) {
  return guarded([&]() { need(h, "handle"); h->e->uploadInputs(n, spatial, global, symmetry); });
}
int kb_forward_resident(kb_handle* h, int n) {
  return guarded([&]() { need(h, "handle"); h->e->forwardResident(n); });
}
int kb_download_outputs(kb_handle* h, int n, float* policy, float* policyPass, float* value, float* scoreValue, float* ownership) {
  return guarded([&]() { need(h, "handle"); h->e->downloadOutputs(n, policy, policyPass, value, scoreValue, ownership); });
}
int kb_forward_host(
  kb_handle* h, int n, const float* spatial, const float* global, const int32_t* symmetry,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership) {
  return guarded([&]() {
    need(h, "handle");
    h->e->uploadInputs(n, spatial, global, symmetry);
    h->e->forwardResident(n);
    h->e->downloadOutputs(n, policy, policyPass, value, scoreValue, ownership);
  });
}
int kb_upload_inputs_meta(kb_handle* h, int n, const float* spatial, const float* global, const float* meta, const int32_t* symmetry) {
  return guarded([&]() { need(h, "handle"); h->e->uploadInputs(n, spatial, global, symmetry, meta); });
}
int kb_forward_host_meta(
  kb_handle* h, int n, const float* spatial, const float* global, const float* meta, const int32_t* symmetry,
  float* policy, float* policyPass, float* value, float* scoreValue, float* ownership) {
  return guarded([&]() {
    need(h, "handle");
    h->e->uploadInputs(n, spatial, global, symmetry, meta);
    h->e->forwardResident(n);
    h->e->downloadOutputs(n, policy, policyPass, value, scoreValue, ownership);
  });
}
int kb_time_forward_resident(kb_handle* h, int n, int iters, float* msPerIter) {
  return guarded([&]() { need(h, "handle"); need(msPerIter, "msPerIter"); *msPerIter = h->e->timeForwardResident(n, iters); });
}

int kb_time_forward_steps(kb_handle* h, int n, int steps, size_t flushBytes, float* msEach) {
  return guarded([&]() { need(h, "handle"); need(msEach, "msEach"); h->e->timeForwardSteps(n, steps, flushBytes, msEach); });
}

int kb_profile_enable(kb_handle* h, int enabled) {
  return guarded([&]() { need(h, "handle"); h->e->profileEnable(enabled != 0); });
}
int kb_profile_reset(kb_handle* h) {
  return guarded([&]() { need(h, "handle"); h->e->profileReset(); });
}
int kb_profile_read(kb_handle* h, kb_profile_entry* entries, int cap, int* count) {
  return guarded([&]() {
    need(h, "handle"); need(entries, "entries"); need(count, "count");
    std::vector<kb::OpClass> tmp(cap > 0 ? cap : 0);
    int k = h->e->profileRead(tmp.data(), cap);
    for(int i = 0; i < k; i++) {
      std::memset(entries[i].name, 0, sizeof(entries[i].name));
      std::strncpy(entries[i].name, tmp[i].name.c_str(), sizeof(entries[i].name) - 1);
      entries[i].launches = tmp[i].launches;
      entries[i].ms = tmp[i].ms;
      entries[i].flops = tmp[i].flops;
      entries[i].bytes = tmp[i].bytes;
    }
    *count = k;
  });
}
int kb_launches_per_forward(const kb_handle* h, int n, int* launches) {
  return guarded([&]() { need(h, "handle"); need(launches, "launches"); *launches = h->e->launchesPerForward(n); });
}
int kb_debug_read_trunk(kb_handle* h, int n, float* trunkOut) {
  return guarded([&]() { need(h, "handle"); h->e->readTrunk(n, trunkOut); });
}

int kb_host_alloc(size_t bytes, void** out) {
  if(out) *out = nullptr;
  return guarded([&]() {
    need(out, "out");
    kb::cudaCheck(cudaHostAlloc(out, bytes, cudaHostAllocPortable), "cudaHostAlloc");
  });
}
void kb_host_free(void* p) {
  if(p) cudaFreeHost(p);
}

int kb_eval_layer(
  const void* blob, size_t nbytes, int device, int precision, int n, int nnXLen, int nnYLen,
  const float* in, const float* mask, float* out) {
  return guarded([&]() {
    kb::Engine e(blob, nbytes, device, n, nnXLen, nnYLen, precision);
    e.evalLayer(in, mask, out);
  });
}

}  // extern "C"
