// Provider probing and adapter / GID / port selection without a verbs library.
//
// The reference answers "which HCA belongs to this GPU, which GID addresses the
// fabric, what does the local end of an RC path look like" by opening an
// ibv_context (src/runtime/core/aboleth_device_select.cu; C ABI at
// include/aboleth/runtime_c.h:131-171), and resolves provider libraries at first
// use through dlopen shims so that none is a link-time dependency
// (src/runtime/dl/*, src/runtime/provider_caps.cpp:37-69).
//
// This build has no verbs code path, so the same questions are answered from what
// the kernel publishes under /sys: /sys/class/infiniband/<hca>/device is the PCI
// function, ports/<n>/{link_layer,lid,state} describe a port, ports/<n>/gids/<i>
// and gid_attrs/types/<i> are the GID table.  The answers are the ones a verbs
// client on the same machine would get, and an external client that opens its own
// queue pair can use them.  Provider libraries are only ever dlopen'ed: a probe
// reports a provider when its library resolves (with one marker symbol) AND the
// machine presents a device for it.
//
// Environment: ABOLETH_HCA, ABOLETH_PORT, ABOLETH_GID_INDEX, ABOLETH_PATH_MTU as in
// the reference; ABOLETH_SYSFS_ROOT (default /sys) and ABOLETH_GPU_PCI_BUS_IDS (a
// comma-separated bus id per CUDA ordinal) let a machine without adapters or GPUs
// exercise the selection; ABOLETH_DL_<NAME> replaces a provider's library name.
#include <algorithm>
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include <dirent.h>
#include <dlfcn.h>
#include <limits.h>
#include <unistd.h>

#include <cuda_runtime.h>

#include "aboleth/runtime_c.h"

extern "C" void ab200_set_last_error(const char *message);

namespace {

int fail(const std::string &message) {
    ab200_set_last_error(message.c_str());
    return -1;
}

std::string env(const char *name) {
    const char *value = std::getenv(name);
    return value ? value : "";
}

std::string sysfs_root() {
    const std::string root = env("ABOLETH_SYSFS_ROOT");
    return root.empty() ? "/sys" : root;
}

std::string read_line(const std::string &path) {
    std::ifstream in(path);
    std::string line;
    std::getline(in, line);
    while (!line.empty() && std::isspace(static_cast<unsigned char>(line.back())))
        line.pop_back();
    return line;
}

std::vector<std::string> list_dir(const std::string &path) {
    std::vector<std::string> names;
    if (DIR *dir = opendir(path.c_str())) {
        while (dirent *entry = readdir(dir))
            if (entry->d_name[0] != '.')
                names.push_back(entry->d_name);
        closedir(dir);
    }
    std::sort(names.begin(), names.end());
    return names;
}

std::string real_path(const std::string &path) {
    char resolved[PATH_MAX];
    return realpath(path.c_str(), resolved) ? std::string(resolved) : std::string();
}

std::string base_name(const std::string &path) {
    const std::size_t slash = path.find_last_of('/');
    return slash == std::string::npos ? path : path.substr(slash + 1);
}

struct Hca {
    std::string name, pci_path, driver;
    bool mlx5() const { return driver == "mlx5_core" || name.rfind("mlx5_", 0) == 0; }
    bool efa() const { return driver == "efa" || name.rfind("efa_", 0) == 0 || name.rfind("rdmap", 0) == 0; }
    bool ionic() const { return driver == "ionic_rdma" || name.rfind("ionic_", 0) == 0; }
};

std::vector<Hca> list_hcas() {
    std::vector<Hca> out;
    const std::string base = sysfs_root() + "/class/infiniband";
    for (const std::string &name : list_dir(base)) {
        Hca hca;
        hca.name = name;
        hca.pci_path = real_path(base + "/" + name + "/device");
        hca.driver = base_name(real_path(base + "/" + name + "/device/driver"));
        out.push_back(hca);
    }
    return out;
}

std::vector<std::string> components(const std::string &path) {
    std::vector<std::string> parts;
    std::stringstream in(path);
    for (std::string part; std::getline(in, part, '/');)
        if (!part.empty())
            parts.push_back(part);
    return parts;
}

// Number of leading path components two PCI functions share: functions behind
// the same switch share more of the path than functions on different root ports.
std::size_t shared_depth(const std::string &a, const std::string &b) {
    const auto pa = components(a), pb = components(b);
    std::size_t n = 0;
    while (n < pa.size() && n < pb.size() && pa[n] == pb[n])
        ++n;
    return n;
}

std::string lower(std::string text) {
    std::transform(text.begin(), text.end(), text.begin(), [](unsigned char c) { return std::tolower(c); });
    return text;
}

std::string gpu_pci_path(int gpu_index, std::string &error) {
    std::string bus_id;
    const std::string listed = env("ABOLETH_GPU_PCI_BUS_IDS");
    if (!listed.empty()) {
        std::stringstream in(listed);
        std::string item;
        for (int i = 0; std::getline(in, item, ','); ++i)
            if (i == gpu_index)
                bus_id = item;
        if (bus_id.empty()) {
            error = "ABOLETH_GPU_PCI_BUS_IDS names no bus id for CUDA ordinal " + std::to_string(gpu_index);
            return "";
        }
    } else {
        char buffer[32] = {0};
        if (cudaDeviceGetPCIBusId(buffer, sizeof(buffer), gpu_index) != cudaSuccess) {
            cudaGetLastError();
            error = "CUDA ordinal " + std::to_string(gpu_index) + " has no PCI bus id (is it visible?)";
            return "";
        }
        bus_id = buffer;
    }
    const std::string path = real_path(sysfs_root() + "/bus/pci/devices/" + lower(bus_id));
    if (path.empty())
        error = "PCI function " + bus_id + " is not listed under " + sysfs_root() + "/bus/pci/devices";
    return path;
}

int chosen_port(int port) {
    if (port > 0)
        return port;
    const std::string named = env("ABOLETH_PORT");
    return named.empty() ? 1 : std::atoi(named.c_str());
}

std::string port_dir(const std::string &device, int port) {
    return sysfs_root() + "/class/infiniband/" + device + "/ports/" + std::to_string(port);
}

bool resolve_device(const char *device_name, std::string &name) {
    if (device_name != nullptr && device_name[0] != '\0') {
        name = device_name;
    } else {
        char buffer[64];
        if (aboleth_runtime_select_device(-1, buffer, sizeof(buffer)) != 0)
            return false;
        name = buffer;
    }
    if (list_dir(sysfs_root() + "/class/infiniband/" + name + "/ports").empty()) {
        fail("adapter '" + name + "' is not present (no ports under " + sysfs_root() + "/class/infiniband)");
        return false;
    }
    return true;
}

bool parse_gid(const std::string &text, std::uint8_t out[16]) {
    // "fe80:0000:0000:0000:0002:c903:00ab:cdef": eight groups of four hex digits.
    std::stringstream in(text);
    std::string group;
    int n = 0;
    while (std::getline(in, group, ':')) {
        if (n == 8 || group.size() != 4 || group.find_first_not_of("0123456789abcdefABCDEF") != std::string::npos)
            return false;
        const unsigned long value = std::strtoul(group.c_str(), nullptr, 16);
        out[2 * n] = static_cast<std::uint8_t>(value >> 8);
        out[2 * n + 1] = static_cast<std::uint8_t>(value & 0xff);
        ++n;
    }
    return n == 8;
}

bool gid_is_zero(const std::uint8_t gid[16]) {
    for (int i = 0; i < 16; ++i)
        if (gid[i] != 0)
            return false;
    return true;
}

bool gid_is_ipv4_mapped(const std::uint8_t gid[16]) {
    for (int i = 0; i < 10; ++i)
        if (gid[i] != 0)
            return false;
    return gid[10] == 0xff && gid[11] == 0xff;
}

// ibv_mtu enumerators: 1 = 256 ... 5 = 4096 bytes.
std::uint32_t mtu_enum_at_most(long bytes) {
    std::uint32_t value = 1;
    for (long size = 512; size <= 4096 && size <= bytes; size *= 2)
        ++value;
    return value;
}

bool library_resolves(const char *override_env, const char *soname, const char *marker) {
    const std::string named = env(override_env);
    void *handle = dlopen(named.empty() ? soname : named.c_str(), RTLD_LAZY | RTLD_LOCAL);
    if (handle == nullptr)
        return false;
    const bool ok = dlsym(handle, marker) != nullptr;
    dlclose(handle);
    return ok;
}

}  // namespace

extern "C" {

std::uint32_t ab200_probe_providers() {
    const std::vector<Hca> hcas = list_hcas();
    const auto any = [&](bool (Hca::*is)() const) {
        return std::any_of(hcas.begin(), hcas.end(), [&](const Hca &h) { return (h.*is)(); });
    };
    std::uint32_t bits = 0;
    const bool verbs = library_resolves("ABOLETH_DL_IBVERBS", "libibverbs.so.1", "ibv_get_device_list");
    if (verbs && !hcas.empty())
        bits |= kAbolethProviderVerbs;
    if (verbs && any(&Hca::mlx5) && library_resolves("ABOLETH_DL_MLX5", "libmlx5.so.1", "mlx5dv_init_obj"))
        bits |= kAbolethProviderMlx5;
    if (verbs && any(&Hca::efa) && library_resolves("ABOLETH_DL_EFA", "libefa.so.1", "efadv_query_device"))
        bits |= kAbolethProviderEfa;
    if (any(&Hca::efa) && library_resolves("ABOLETH_DL_FABRIC", "libfabric.so.1", "fi_getinfo"))
        bits |= kAbolethProviderLibfabric;
    if (library_resolves("ABOLETH_DL_CUDA", "libcuda.so.1", "cuInit")) {
        int gpus = 0;
        if (cudaGetDeviceCount(&gpus) != cudaSuccess) {
            cudaGetLastError();
            gpus = 0;
        }
        if (gpus > 0)
            bits |= kAbolethProviderCuda;
    }
    if (!list_dir(sysfs_root() + "/class/kfd/kfd/topology/nodes").empty() &&
        library_resolves("ABOLETH_DL_HIP", "libamdhip64.so", "hipInit"))
        bits |= kAbolethProviderHip;
    if (verbs && any(&Hca::ionic) && library_resolves("ABOLETH_DL_IONIC", "libionic.so.1", "ionic_dv_ctx_get_udma_count"))
        bits |= kAbolethProviderIonic;
    return bits;
}

int aboleth_runtime_select_device(int gpu_index, char *name_out, std::size_t name_capacity) {
    if (name_out == nullptr || name_capacity == 0)
        return fail("select_device needs a buffer for the adapter's name");
    std::vector<Hca> candidates;
    for (const Hca &hca : list_hcas())
        if (hca.mlx5())
            candidates.push_back(hca);
    std::string chosen;
    const std::string forced = env("ABOLETH_HCA");
    if (!forced.empty()) {
        const std::vector<Hca> all = list_hcas();
        if (std::none_of(all.begin(), all.end(), [&](const Hca &h) { return h.name == forced; }))
            return fail("ABOLETH_HCA names '" + forced + "', which is not under " + sysfs_root() +
                        "/class/infiniband");
        chosen = forced;
    } else if (candidates.empty()) {
        return fail("no mlx5 adapter is present under " + sysfs_root() + "/class/infiniband");
    } else if (gpu_index < 0) {
        chosen = candidates.front().name;  // topology-free default: first in name order
    } else {
        std::string error;
        const std::string gpu = gpu_pci_path(gpu_index, error);
        if (gpu.empty())
            return fail(error);
        std::size_t best = 0;
        for (const Hca &hca : candidates) {
            const std::size_t depth = shared_depth(gpu, hca.pci_path);
            if (chosen.empty() || depth > best) {  // ties keep the first in name order
                chosen = hca.name;
                best = depth;
            }
        }
    }
    if (chosen.size() + 1 > name_capacity)
        return fail("the adapter's name needs " + std::to_string(chosen.size() + 1) + " bytes");
    std::memcpy(name_out, chosen.c_str(), chosen.size() + 1);
    return 0;
}

int aboleth_runtime_select_gid_index(const char *device_name, int port) {
    std::string device;
    if (!resolve_device(device_name, device))
        return -1;
    const std::string dir = port_dir(device, chosen_port(port));
    if (read_line(dir + "/link_layer").empty())
        return fail("adapter '" + device + "' has no port " + std::to_string(chosen_port(port)));
    const std::string forced = env("ABOLETH_GID_INDEX");
    if (!forced.empty())
        return std::atoi(forced.c_str());
    if (read_line(dir + "/link_layer") == "InfiniBand")
        return 0;
    // RoCE: a v2 entry, the IPv4-mapped one first; then any populated entry.
    int v2 = -1, v2_ipv4 = -1, populated = -1;
    std::vector<int> indices;
    for (const std::string &name : list_dir(dir + "/gids"))
        indices.push_back(std::atoi(name.c_str()));
    std::sort(indices.begin(), indices.end());
    for (int index : indices) {
        std::uint8_t gid[16];
        if (!parse_gid(read_line(dir + "/gids/" + std::to_string(index)), gid) || gid_is_zero(gid))
            continue;
        if (populated < 0)
            populated = index;
        if (read_line(dir + "/gid_attrs/types/" + std::to_string(index)) == "RoCE v2") {
            if (v2 < 0)
                v2 = index;
            if (v2_ipv4 < 0 && gid_is_ipv4_mapped(gid))
                v2_ipv4 = index;
        }
    }
    const int index = v2_ipv4 >= 0 ? v2_ipv4 : (v2 >= 0 ? v2 : populated);
    if (index < 0)
        return fail("port " + std::to_string(chosen_port(port)) + " of '" + device + "' has no populated GID");
    return index;
}

int aboleth_runtime_query_port_address(const char *device_name, int port, std::uint16_t *lid_out,
                                       std::uint8_t *link_layer_out, std::uint8_t *gid_out16,
                                       int *gid_index_out, std::uint32_t *path_mtu_out) {
    std::string device;
    if (!resolve_device(device_name, device))
        return -1;
    const int gid_index = aboleth_runtime_select_gid_index(device.c_str(), port);
    if (gid_index < 0)
        return -1;
    const std::string dir = port_dir(device, chosen_port(port));
    const bool infiniband = read_line(dir + "/link_layer") == "InfiniBand";
    std::uint8_t gid[16] = {0};
    if (!parse_gid(read_line(dir + "/gids/" + std::to_string(gid_index)), gid))
        return fail("GID " + std::to_string(gid_index) + " of '" + device + "' cannot be read");
    if (lid_out)
        *lid_out = static_cast<std::uint16_t>(std::strtoul(read_line(dir + "/lid").c_str(), nullptr, 0));
    if (link_layer_out)
        *link_layer_out = infiniband ? 1 : 2;  // IBV_LINK_LAYER_INFINIBAND / _ETHERNET
    if (gid_out16)
        std::memcpy(gid_out16, gid, 16);
    if (gid_index_out)
        *gid_index_out = gid_index;
    if (path_mtu_out) {
        long bytes = infiniband ? 4096 : 1024;
        if (!infiniband) {
            // A RoCE path carries at most the netdev's MTU minus the headers.
            const std::string netdev = read_line(dir + "/gid_attrs/ndevs/" + std::to_string(gid_index));
            const std::string mtu = netdev.empty() ? "" : read_line(sysfs_root() + "/class/net/" + netdev + "/mtu");
            if (!mtu.empty())
                bytes = std::atol(mtu.c_str()) - 58;
        }
        const std::string forced = env("ABOLETH_PATH_MTU");
        if (!forced.empty()) {
            const long asked = std::atol(forced.c_str());
            if (asked != 256 && asked != 512 && asked != 1024 && asked != 2048 && asked != 4096)
                return fail("ABOLETH_PATH_MTU must be 256, 512, 1024, 2048 or 4096");
            bytes = std::min(bytes, asked);
        }
        *path_mtu_out = mtu_enum_at_most(std::max(bytes, 256l));
    }
    return 0;
}

}  // extern "C"
