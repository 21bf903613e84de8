// Network backend choice: an external plugin (NCCL_NET_PLUGIN) exporting ncclNetPlugin_v12 (or an
// earlier table down to v8, wrapped by net_compat.cc), or the built-in TCP backend. NCCL_NET=<name> insists on one backend by name.
// Reference parity: src/plugin/net.cc:60-495 (external first, then internal backends; name match
// against NCCL_NET), src/plugin/net/net_v12.cc.
#include <mutex>

#include "../transport/net.h"
#include "plugin.h"
#include "plugin/nccl_gin.h"

namespace b200 {

static std::once_flag gNetOnce;
static ncclNet_t* gNet = nullptr;
static bool gNetExternal = false;
static ncclCollNet_t* gCollNet = nullptr;
// A table for GPU-initiated networking in the network plugin library: initialised once to learn what it offers (devices,
// signal kinds); this build has no network to hand it (one NVLink domain), so it is reported and finalised.
static GinPluginInfo gGin;

ncclResult_t netSelect(ncclNet_t** net, bool* external) {
  std::call_once(gNetOnce, [] {
    const char* wantName = getEnv("NCCL_NET");
    std::string resolved;
    void* lib = pluginOpen(PLUGIN_NET, &resolved);
    ncclNet_t* ext = lib ? (ncclNet_t*)pluginSymbol(lib, NCCL_NET_PLUGIN_SYMBOL) : nullptr;
    if (lib && !ext) {
      int version = 0;
      ext = netCompatWrap(lib, &version);   // v11 ... v8 behind an adapter with the current signature
      if (ext) INFO(SUB_NET | SUB_INIT, "net plugin %s speaks interface v%d: loaded through an adapter", resolved.c_str(), version);
    }
    gCollNet = lib ? (ncclCollNet_t*)pluginSymbol(lib, NCCL_COLLNET_PLUGIN_SYMBOL) : nullptr;
    if (gCollNet) INFO(SUB_NET | SUB_INIT, "net plugin %s offers the collective network %s", resolved.c_str(), gCollNet->name ? gCollNet->name : "?");
    if (ncclGin_t* gin = lib ? (ncclGin_t*)pluginSymbol(lib, NCCL_GIN_PLUGIN_SYMBOL) : nullptr) {
      void* gctx = nullptr;
      int ndev = 0;
      ncclGinProperties_t gp = {false, false};
      if (gin->init && gin->init(&gctx, 0, pluginLogger) == ncclSuccess) {
        if (gin->devices) gin->devices(&ndev);
        if (gin->getGinProperties) gin->getGinProperties(&gp);
        if (gin->finalize) gin->finalize(gctx);
        gGin.present = true;
        gGin.name = gin->name ? gin->name : "?";
        gGin.devices = ndev;
        gGin.strongSignals = gp.supportsStrongSignals;
        gGin.vaSignals = gp.supportsVASignals;
        INFO(SUB_NET | SUB_INIT, "net plugin %s offers GPU-initiated networking %s: %d device(s), strong signals %d, VA signals %d; not used: this build moves GPU-initiated traffic inside one NVLink domain",
             resolved.c_str(), gGin.name.c_str(), ndev, (int)gp.supportsStrongSignals, (int)gp.supportsVASignals);
      } else {
        WARN("net plugin %s: %s failed to initialise", resolved.c_str(), NCCL_GIN_PLUGIN_SYMBOL);
      }
    }
    if (lib && !ext && gCollNet) INFO(SUB_NET | SUB_INIT, "net plugin %s has no point-to-point table (%s): point-to-point traffic stays on the built-in backend", resolved.c_str(), NCCL_NET_PLUGIN_SYMBOL);
    else if (lib && !ext) WARN("net plugin %s exports none of ncclNetPlugin_v12 ... ncclNetPlugin_v8; using the built-in backend", resolved.c_str());
    if (ext && wantName && *wantName && strcasecmp(wantName, ext->name) != 0 &&
        (strcasecmp(wantName, netSocketBackend.name) == 0 || strcasecmp(wantName, netIbBackend.name) == 0)) ext = nullptr;
    if (ext) {
      int ndev = 0;
      void* ctx = nullptr;
      ncclNetCommConfig_t cfg = {NCCL_NET_TRAFFIC_CLASS_UNDEF};
      if (ext->init(&ctx, 0, &cfg, pluginLogger, nullptr) == ncclSuccess && ext->devices(&ndev) == ncclSuccess && ndev > 0) {
        if (ext->finalize) ext->finalize(ctx);
        gNet = ext;
        gNetExternal = true;
        INFO(SUB_NET | SUB_INIT, "network backend: plugin %s (%s), %d device(s)", ext->name, resolved.c_str(), ndev);
        return;
      }
      WARN("net plugin %s found no usable device; using the built-in backend", ext->name);
    }
    const bool wantSocket = wantName && *wantName && strcasecmp(wantName, netSocketBackend.name) == 0;
    if (!wantSocket) {
      int ndev = 0;
      void* ctx = nullptr;
      ncclNetCommConfig_t cfg = {NCCL_NET_TRAFFIC_CLASS_UNDEF};
      if (netIbBackend.init(&ctx, 0, &cfg, pluginLogger, nullptr) == ncclSuccess && netIbBackend.devices(&ndev) == ncclSuccess && ndev > 0) {
        gNet = &netIbBackend;
        INFO(SUB_NET | SUB_INIT, "network backend: built-in %s, %d device(s)", netIbBackend.name, ndev);
        return;
      }
    }
    if (wantName && *wantName && !wantSocket)
      WARN("NCCL_NET=%s does not match any available backend; using %s", wantName, netSocketBackend.name);
    gNet = &netSocketBackend;
    INFO(SUB_NET | SUB_INIT, "network backend: built-in %s", gNet->name);
  });
  *net = gNet;
  if (external) *external = gNetExternal;
  return gNet ? ncclSuccess : ncclInternalError;
}

const GinPluginInfo* netGinPluginInfo() {
  ncclNet_t* net;
  if (netSelect(&net, nullptr) != ncclSuccess) return nullptr;
  return &gGin;
}

ncclCollNet_t* netCollNetTable() {
  ncclNet_t* net;
  if (netSelect(&net, nullptr) != ncclSuccess) return nullptr;
  return gCollNet;
}

}  // namespace b200
