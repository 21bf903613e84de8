// Topology as an XML tree: parser, writer, machine probe and fusion of per-process views.
// Shape of the document (same element and attribute names as the reference's dumps, so that a
// file written by either library loads in the other):
//   <system version="1">
//     <cpu numaid="0" affinity="..." arch="x86_64" vendor="..." >
//       <pci busid="0000:17:00.0" class="0x060400" link_speed="32.0 GT/s PCIe" link_width="16">
//         <pci busid="0000:19:00.0" class="0x030200" ...>
//           <gpu dev="0" sm="100" rank="0" gdr="1">
//             <nvlink target="0000:05:00.0" count="18" tclass="0x068000"/>
//     ...
//       <nic> <net name="mlx5_0" dev="0" speed="400000" port="1" gdr="1"/> </nic>
// Reference parity: src/graph/xml.cc (:38-256 parser, :275-304 dump, :306-342 fuse, :471 CPU,
// :589 PCI from sysfs, :894 GPU / NVLink, :1098 NICs).
#include <dirent.h>
#include <dlfcn.h>
#include <limits.h>
#include <stdio.h>
#include <unistd.h>

#include <fstream>
#include <sstream>

#include "../core/nvmlwrap.h"
#include "topo.h"

namespace b200 {

const char* XmlNode::attr(const char* key) const {
  for (auto& a : attrs) if (a.first == key) return a.second.c_str();
  return nullptr;
}
void XmlNode::setAttr(const std::string& key, const std::string& value) {
  for (auto& a : attrs) if (a.first == key) { a.second = value; return; }
  attrs.push_back({key, value});
}
int XmlNode::attrInt(const char* key, int deflt) const {
  const char* v = attr(key);
  return v ? (int)strtol(v, nullptr, 0) : deflt;
}
double XmlNode::attrFloat(const char* key, double deflt) const {
  const char* v = attr(key);
  return v ? strtod(v, nullptr) : deflt;
}
XmlNode* XmlNode::addSub(const std::string& n) {
  XmlNode* s = new XmlNode;
  s->name = n;
  s->parent = this;
  subs.push_back(s);
  return s;
}
XmlNode* XmlNode::findSub(const char* n, const char* k, const char* v) {
  for (auto* s : subs) {
    if (s->name != n) continue;
    if (!k) return s;
    const char* a = s->attr(k);
    if (a && !strcmp(a, v)) return s;
  }
  return nullptr;
}

// ---------------------------------------------------------------- parser
struct XmlParser {
  const std::string& t;
  size_t p = 0;
  std::string err;
  explicit XmlParser(const std::string& text) : t(text) {}
  void ws() { while (p < t.size() && isspace((unsigned char)t[p])) ++p; }
  bool skipMisc() {
    for (;;) {
      ws();
      if (t.compare(p, 4, "<!--") == 0) { size_t e = t.find("-->", p); if (e == std::string::npos) return false; p = e + 3; continue; }
      if (t.compare(p, 2, "<?") == 0) { size_t e = t.find("?>", p); if (e == std::string::npos) return false; p = e + 2; continue; }
      return true;
    }
  }
  std::string ident() {
    size_t b = p;
    while (p < t.size() && (isalnum((unsigned char)t[p]) || t[p] == '_' || t[p] == '-' || t[p] == ':' || t[p] == '.')) ++p;
    return t.substr(b, p - b);
  }
  XmlNode* element(XmlNode* parent) {
    if (!skipMisc() || p >= t.size() || t[p] != '<') { err = "expected '<'"; return nullptr; }
    ++p;
    XmlNode* n = new XmlNode;
    n->parent = parent;
    n->name = ident();
    if (n->name.empty()) { err = "empty element name"; delete n; return nullptr; }
    for (;;) {
      ws();
      if (p >= t.size()) { err = "unterminated element"; delete n; return nullptr; }
      if (t[p] == '/') {
        if (p + 1 < t.size() && t[p + 1] == '>') { p += 2; return n; }
        err = "stray '/'"; delete n; return nullptr;
      }
      if (t[p] == '>') { ++p; break; }
      std::string k = ident();
      ws();
      if (k.empty() || p >= t.size() || t[p] != '=') { err = "malformed attribute in <" + n->name + ">"; delete n; return nullptr; }
      ++p;
      ws();
      if (p >= t.size() || (t[p] != '"' && t[p] != '\'')) { err = "attribute value must be quoted"; delete n; return nullptr; }
      char q = t[p++];
      size_t e = t.find(q, p);
      if (e == std::string::npos) { err = "unterminated attribute value"; delete n; return nullptr; }
      n->attrs.push_back({k, t.substr(p, e - p)});
      p = e + 1;
    }
    // children until the closing tag
    for (;;) {
      if (!skipMisc()) { err = "unterminated comment"; delete n; return nullptr; }
      if (p >= t.size()) { err = "missing </" + n->name + ">"; delete n; return nullptr; }
      if (t[p] != '<') { ++p; continue; }   // text content is ignored
      if (p + 1 < t.size() && t[p + 1] == '/') {
        p += 2;
        std::string c = ident();
        ws();
        if (c != n->name || p >= t.size() || t[p] != '>') { err = "mismatched </" + c + "> for <" + n->name + ">"; delete n; return nullptr; }
        ++p;
        return n;
      }
      XmlNode* s = element(n);
      if (!s) { delete n; return nullptr; }
      n->subs.push_back(s);
    }
  }
};

XmlNode* xmlParse(const std::string& text, std::string* err) {
  XmlParser ps(text);
  XmlNode* root = ps.element(nullptr);
  if (!root && err) *err = ps.err;
  return root;
}

XmlNode* xmlLoadFile(const char* path, std::string* err) {
  std::ifstream f(path);
  if (!f) { if (err) *err = std::string("cannot open ") + path; return nullptr; }
  std::stringstream ss;
  ss << f.rdbuf();
  return xmlParse(ss.str(), err);
}

std::string xmlDump(const XmlNode* n, int indent) {
  std::string pad(indent * 2, ' ');
  std::string s = pad + "<" + n->name;
  for (auto& a : n->attrs) s += " " + a.first + "=\"" + a.second + "\"";
  if (n->subs.empty()) return s + "/>\n";
  s += ">\n";
  for (auto* c : n->subs) s += xmlDump(c, indent + 1);
  return s + pad + "</" + n->name + ">\n";
}

// ---------------------------------------------------------------- machine probe
static std::string readFile(const std::string& path) {
  std::ifstream f(path);
  std::string s;
  if (f) std::getline(f, s);
  while (!s.empty() && (s.back() == '\n' || s.back() == ' ')) s.pop_back();
  return s;
}

static std::string lower(std::string s) {
  for (auto& c : s) c = (char)tolower((unsigned char)c);
  return s;
}

// Walks /sys/bus/pci/devices/<busid> upward and creates the <pci> chain under the right <cpu>.
static XmlNode* pciChain(XmlNode* system, const std::string& busId) {
  char real[PATH_MAX];
  std::string link = "/sys/bus/pci/devices/" + busId;
  std::vector<std::string> chain;   // root port first
  int numa = -1;
  if (realpath(link.c_str(), real)) {
    // .../pci0000:16/0000:16:01.0/0000:17:00.0/0000:19:00.0
    std::string path(real);
    size_t pos = 0;
    while ((pos = path.find('/', pos)) != std::string::npos) {
      size_t e = path.find('/', pos + 1);
      std::string comp = path.substr(pos + 1, e == std::string::npos ? std::string::npos : e - pos - 1);
      if (comp.size() == 12 && comp[4] == ':' && comp[7] == ':' && comp[10] == '.') chain.push_back(comp);
      pos = pos + 1;
    }
    std::string nn = readFile(link + "/numa_node");
    if (!nn.empty()) numa = atoi(nn.c_str());
  } else {
    chain.push_back(busId);
  }
  if (numa < 0) numa = 0;
  XmlNode* cpu = system->findSub("cpu", "numaid", std::to_string(numa).c_str());
  if (!cpu) {
    cpu = system->addSub("cpu");
    cpu->setAttr("numaid", std::to_string(numa));
    cpu->setAttr("affinity", readFile("/sys/devices/system/node/node" + std::to_string(numa) + "/cpumap"));
#if defined(__x86_64__)
    cpu->setAttr("arch", "x86_64");
#elif defined(__aarch64__)
    cpu->setAttr("arch", "arm64");
#else
    cpu->setAttr("arch", "unknown");
#endif
    std::ifstream ci("/proc/cpuinfo");
    std::string line;
    while (std::getline(ci, line)) {
      if (line.compare(0, 9, "vendor_id") == 0) { cpu->setAttr("vendor", line.substr(line.find(':') + 2)); break; }
    }
  }
  XmlNode* cur = cpu;
  // keep only switches (bridges) and the device itself, like the reference's flattened tree
  for (size_t i = 0; i < chain.size(); ++i) {
    XmlNode* s = cur->findSub("pci", "busid", chain[i].c_str());
    if (!s) {
      s = cur->addSub("pci");
      s->setAttr("busid", chain[i]);
      std::string dev = "/sys/bus/pci/devices/" + chain[i];
      std::string cls = readFile(dev + "/class");
      s->setAttr("class", cls.empty() ? "0x000000" : cls);
      s->setAttr("vendor", readFile(dev + "/vendor"));
      s->setAttr("device", readFile(dev + "/device"));
      std::string sp = readFile(dev + "/max_link_speed"), wd = readFile(dev + "/max_link_width");
      s->setAttr("link_speed", sp.empty() ? "32.0 GT/s PCIe" : sp);
      s->setAttr("link_width", wd.empty() ? "16" : wd);
    }
    cur = s;
  }
  return cur;
}

XmlNode* xmlFromSystem() {
  XmlNode* system = new XmlNode;
  system->name = "system";
  system->setAttr("version", "1");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess) { (void)cudaGetLastError(); ndev = 0; }
  std::vector<std::string> busIds(ndev);
  for (int d = 0; d < ndev; ++d) {
    char b[32] = "";
    cudaDeviceGetPCIBusId(b, sizeof(b), d);
    busIds[d] = lower(b);
  }
  const NvmlApi* nvml = nvmlApi();
  for (int d = 0; d < ndev; ++d) {
    XmlNode* pci = pciChain(system, busIds[d]);
    XmlNode* gpu = pci->findSub("gpu");
    if (!gpu) gpu = pci->addSub("gpu");
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, d);
    gpu->setAttr("dev", std::to_string(d));
    gpu->setAttr("sm", std::to_string(prop.major * 10 + prop.minor));
    gpu->setAttr("gdr", "1");
    // NVLinks: NVML tells the remote end of every active link; without NVML, fall back to the
    // peer-access matrix (every reachable peer counts as connected through a switch).
    std::map<std::string, int> remotes;
    bool viaNvml = false;
    if (nvml) {
      nvmlDevice_t h;
      if (nvml->deviceGetHandleByPciBusId(busIds[d].c_str(), &h) == 0) {
        viaNvml = true;
        for (unsigned l = 0; l < 18; ++l) {
          unsigned active = 0;
          if (nvml->deviceGetNvLinkState(h, l, &active) != 0 || !active) continue;
          nvmlPciInfo_t pi;
          if (nvml->deviceGetNvLinkRemotePciInfo(h, l, &pi) != 0) continue;
          remotes[lower(pi.busId)]++;
        }
      }
    }
    if (!viaNvml) {
      int peers = 0;
      for (int o = 0; o < ndev; ++o) {
        int can = 0;
        if (o != d && cudaDeviceCanAccessPeer(&can, d, o) == cudaSuccess && can) ++peers;
      }
      (void)cudaGetLastError();
      if (peers) remotes["ffff:ff:ff.0"] = prop.major >= 10 ? 18 : 12;   // a switch
    }
    for (auto& kv : remotes) {
      XmlNode* nl = gpu->addSub("nvlink");
      nl->setAttr("target", kv.first);
      nl->setAttr("count", std::to_string(kv.second));
      bool isGpu = false;
      for (auto& b : busIds) if (b == kv.first) isGpu = true;
      nl->setAttr("tclass", isGpu ? "0x030200" : "0x068000");
    }
  }
  // network devices
  DIR* dir = opendir("/sys/class/net");
  if (dir) {
    int devIdx = 0;
    while (struct dirent* de = readdir(dir)) {
      std::string ifn = de->d_name;
      if (ifn == "." || ifn == ".." || ifn == "lo") continue;
      std::string devLink = "/sys/class/net/" + ifn + "/device";
      char real[PATH_MAX];
      if (!realpath(devLink.c_str(), real)) continue;   // virtual interface
      std::string bus = std::string(real).substr(std::string(real).rfind('/') + 1);
      if (bus.size() != 12) continue;
      XmlNode* pci = pciChain(system, bus);
      XmlNode* nic = pci->findSub("nic");
      if (!nic) nic = pci->addSub("nic");
      XmlNode* net = nic->addSub("net");
      net->setAttr("name", ifn);
      net->setAttr("dev", std::to_string(devIdx++));
      std::string speed = readFile("/sys/class/net/" + ifn + "/speed");
      net->setAttr("speed", speed.empty() || atoi(speed.c_str()) <= 0 ? "10000" : speed);
      net->setAttr("port", "0");
      net->setAttr("gdr", "0");
    }
    closedir(dir);
  }
  if (system->subs.empty()) {
    XmlNode* cpu = system->addSub("cpu");
    cpu->setAttr("numaid", "0");
    cpu->setAttr("arch", "x86_64");
  }
  return system;
}

static void fuseInto(XmlNode* dst, const XmlNode* src) {
  for (auto* s : src->subs) {
    const char* keys[] = {"numaid", "busid", "dev", "name", "target"};
    XmlNode* match = nullptr;
    for (auto* d : dst->subs) {
      if (d->name != s->name) continue;
      bool same = true, compared = false;
      for (const char* k : keys) {
        const char* a = d->attr(k);
        const char* b = s->attr(k);
        if (a && b) { compared = true; if (strcmp(a, b)) same = false; }
      }
      if (same && compared) { match = d; break; }
      if (!compared && s->attrs.empty()) { match = d; break; }
    }
    if (!match) {
      match = dst->addSub(s->name);
      match->attrs = s->attrs;
    } else {
      for (auto& a : s->attrs) if (!match->attr(a.first.c_str())) match->setAttr(a.first, a.second);
    }
    fuseInto(match, s);
  }
}
void xmlFuse(XmlNode* dst, const XmlNode* src) { fuseInto(dst, src); }

}  // namespace b200
