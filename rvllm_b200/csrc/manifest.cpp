// Kernel-artifact catalogue: manifest parsing, trust checks, SHA-256, PTX module loading through
// the CUDA driver API (resolved with dlopen so the library still loads on a machine without a
// driver) and the raw launcher.  Host code only.
#include <dlfcn.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/rvllm_b200.h"
#include "../../include/rvllm_b200_manifest.h"

int rv_fail(int code, const char* fmt, ...);

namespace {

constexpr uint64_t MAX_MANIFEST_BYTES = 1024 * 1024;
constexpr uint64_t MAX_ARTIFACT_BYTES = 512ull * 1024 * 1024;
constexpr size_t MAX_ARTIFACTS = 4096;

// ---- SHA-256 (FIPS 180-4) ---------------------------------------------------------------
struct Sha256 {
    uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint8_t buf[64];
    size_t fill = 0;
    uint64_t total = 0;
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98,
            0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786,
            0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8,
            0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
            0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819,
            0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a,
            0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
            0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++)
            w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
            uint32_t ch = (e & f) ^ (~e & g);
            uint32_t t1 = hh + S1 + ch + K[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
            uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
            uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const uint8_t* p, size_t n) {
        total += n;
        while (n) {
            size_t take = 64 - fill < n ? 64 - fill : n;
            memcpy(buf + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { block(buf); fill = 0; }
        }
    }
    std::string hex() {
        uint64_t bits = total * 8;
        uint8_t pad = 0x80;
        update(&pad, 1);
        uint8_t z = 0;
        while (fill != 56) update(&z, 1);
        uint8_t len[8];
        for (int i = 0; i < 8; i++) len[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(len, 8);
        char out[65];
        for (int i = 0; i < 8; i++) snprintf(out + 8 * i, 9, "%08x", h[i]);
        return std::string(out, 64);
    }
};

std::string sha256_hex(const void* p, size_t n) {
    Sha256 s;
    s.update((const uint8_t*)p, n);
    return s.hex();
}

// ---- a strict JSON reader for exactly the manifest's shape ---------------------------------
struct Json {
    const char* p;
    const char* end;
    std::string err;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool lit(char c) {
        ws();
        if (p < end && *p == c) { p++; return true; }
        return false;
    }
    bool str(std::string& out) {
        ws();
        if (p >= end || *p != '"') return fail("expected a string");
        p++;
        out.clear();
        while (p < end && *p != '"') {
            if ((unsigned char)*p < 0x20) return fail("control character in string");
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                switch (*p) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    default: return fail("unsupported escape in string");
                }
                p++;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool u64(uint64_t& out) {
        ws();
        if (p >= end || *p < '0' || *p > '9') return fail("expected an unsigned integer");
        out = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (out > (UINT64_MAX - 9) / 10) return fail("integer overflows");
            out = out * 10 + (uint64_t)(*p++ - '0');
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("expected an integer");
        return true;
    }
    bool fail(const char* m) {
        if (err.empty()) err = m;
        return false;
    }
};

struct Entry {
    std::string path, sha256, abi;
    uint64_t bytes = 0;
    int kind = -1;
    std::vector<uint8_t> data;
};

bool name_ok(const std::string& s, size_t max) {
    if (s.empty() || s.size() > max) return false;
    for (unsigned char c : s)
        if (!(isalnum(c) || c == '.' || c == '_' || c == '-')) return false;
    return true;
}
bool digest_ok(const std::string& s) {
    if (s.size() != 64) return false;
    for (char c : s)
        if (!((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'))) return false;
    return true;
}
bool ends_with(const std::string& s, const char* suf) {
    size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}
bool path_ok(const std::string& p) {
    if (p.empty() || p[0] == '/' || p.find('\\') != std::string::npos || p.find('\0') != std::string::npos) return false;
    size_t i = 0;
    while (i <= p.size()) {
        size_t j = p.find('/', i);
        if (j == std::string::npos) j = p.size();
        std::string part = p.substr(i, j - i);
        if (part.empty() || part == "." || part == "..") return false;
        i = j + 1;
    }
    return true;
}

bool read_bounded(const std::string& path, uint64_t limit, std::vector<uint8_t>& out, std::string& why) {
    int fd = open(path.c_str(), O_RDONLY | O_CLOEXEC | O_NOFOLLOW);
    if (fd < 0) { why = "cannot open " + path; return false; }
    struct stat st;
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) { close(fd); why = path + " is not a regular file"; return false; }
    if ((uint64_t)st.st_size > limit) { close(fd); why = path + " exceeds the size limit"; return false; }
    out.resize((size_t)st.st_size);
    size_t got = 0;
    while (got < out.size()) {
        ssize_t n = read(fd, out.data() + got, out.size() - got);
        if (n <= 0) { close(fd); why = "short read of " + path; return false; }
        got += (size_t)n;
    }
    close(fd);
    return true;
}

}  // namespace

struct rvllm_manifest {
    std::string revision, arch, dir;
    std::map<std::string, Entry> entries;
};

namespace {

const char* pin_or_env(const char* pin, const char* env) {
    if (pin && *pin) return pin;
    const char* v = getenv(env);
    if (!v) return nullptr;
    while (*v == ' ') v++;
    return *v ? v : nullptr;
}

bool parse_entry(Json& j, Entry& e) {
    if (!j.lit('{')) return j.fail("entry must be an object");
    bool seen[5] = {false, false, false, false, false};
    bool first = true;
    while (!j.lit('}')) {
        if (!first && !j.lit(',')) return j.fail("expected ',' in entry");
        first = false;
        std::string key, val;
        if (!j.str(key) || !j.lit(':')) return j.fail("bad entry field");
        int idx = key == "path" ? 0 : key == "sha256" ? 1 : key == "bytes" ? 2 : key == "kind" ? 3 : key == "abi" ? 4 : -1;
        if (idx < 0) return j.fail("unknown field in entry");
        if (seen[idx]) return j.fail("duplicate field in entry");
        seen[idx] = true;
        if (idx == 2) {
            if (!j.u64(e.bytes)) return false;
        } else {
            if (!j.str(val)) return false;
            if (idx == 0) e.path = val;
            else if (idx == 1) e.sha256 = val;
            else if (idx == 4) e.abi = val;
            else {
                e.kind = val == "ptx" ? 0 : val == "shared_object" ? 1 : -1;
                if (e.kind < 0) return j.fail("unknown artifact kind");
            }
        }
    }
    for (bool s : seen)
        if (!s) return j.fail("entry is missing a field");
    return true;
}

bool parse_manifest(const std::vector<uint8_t>& body, rvllm_manifest& m, std::string& why) {
    Json j{(const char*)body.data(), (const char*)body.data() + body.size(), ""};
    bool seen[3] = {false, false, false};
    bool ok = j.lit('{');
    bool first = true;
    while (ok && !j.lit('}')) {
        if (!first && !j.lit(',')) { ok = j.fail("expected ','"); break; }
        first = false;
        std::string key;
        if (!j.str(key) || !j.lit(':')) { ok = j.fail("bad top-level field"); break; }
        int idx = key == "revision" ? 0 : key == "arch" ? 1 : key == "entries" ? 2 : -1;
        if (idx < 0) { ok = j.fail("unknown top-level field"); break; }
        if (seen[idx]) { ok = j.fail("duplicate top-level field"); break; }
        seen[idx] = true;
        if (idx == 0) ok = j.str(m.revision);
        else if (idx == 1) ok = j.str(m.arch);
        else {
            if (!j.lit('{')) { ok = j.fail("entries must be an object"); break; }
            bool f2 = true;
            while (ok && !j.lit('}')) {
                if (!f2 && !j.lit(',')) { ok = j.fail("expected ',' in entries"); break; }
                f2 = false;
                std::string name;
                Entry e;
                if (!j.str(name) || !j.lit(':') || !parse_entry(j, e)) { ok = false; break; }
                if (m.entries.count(name)) { ok = j.fail("duplicate artifact name"); break; }
                if (m.entries.size() >= MAX_ARTIFACTS) { ok = j.fail("too many artifacts"); break; }
                m.entries.emplace(name, std::move(e));
            }
        }
    }
    if (ok) {
        j.ws();
        if (j.p != j.end) ok = j.fail("trailing data after the manifest object");
    }
    if (ok && !(seen[0] && seen[1] && seen[2])) ok = j.fail("manifest is missing a field");
    if (!ok) why = j.err.empty() ? "malformed manifest" : j.err;
    return ok;
}

}  // namespace

extern "C" {

int rvllm_sha256_hex(const void* data, size_t len, char* out) {
    if ((!data && len) || !out) return rv_fail(RVLLM_E_INVALID, "null argument");
    std::string h = sha256_hex(data, len);
    memcpy(out, h.c_str(), 65);
    return RVLLM_OK;
}

int rvllm_manifest_load_and_verify(rvllm_manifest** out, const char* manifest_path, const char* trusted_sha256,
                                   const char* trusted_revision, const char* trusted_arch) {
    if (!out || !manifest_path) return rv_fail(RVLLM_E_INVALID, "null argument");
    const char* want_sha = pin_or_env(trusted_sha256, "RVLLM_KERNEL_MANIFEST_SHA256");
    const char* want_rev = pin_or_env(trusted_revision, "RVLLM_RELEASE_REVISION");
    const char* want_arch = pin_or_env(trusted_arch, "RVLLM_KERNEL_ARCH");
    if (!want_sha || !want_rev || !want_arch)
        return rv_fail(RVLLM_E_ARTIFACT, "kernel manifest trust: a pin is missing (digest, revision or arch)");
    if (!digest_ok(want_sha)) return rv_fail(RVLLM_E_ARTIFACT, "trusted manifest digest: sha256 must be 64 lowercase hex characters");
    std::vector<uint8_t> body;
    std::string why;
    if (!read_bounded(manifest_path, MAX_MANIFEST_BYTES, body, why)) return rv_fail(RVLLM_E_ARTIFACT, "%s", why.c_str());
    if (sha256_hex(body.data(), body.size()) != want_sha)
        return rv_fail(RVLLM_E_ARTIFACT, "manifest digest does not match the trusted digest");
    rvllm_manifest* m = new rvllm_manifest();
    auto bail = [&](const std::string& msg) {
        delete m;
        return rv_fail(RVLLM_E_ARTIFACT, "%s", msg.c_str());
    };
    if (!parse_manifest(body, *m, why)) return bail("invalid manifest: " + why);
    if (m->revision != want_rev) return bail("revision does not match the trusted revision");
    if (m->arch != want_arch) return bail("architecture does not match the selected target");
    bool hex = m->revision.size() >= 7 && m->revision.size() <= 64;
    for (unsigned char c : m->revision) hex = hex && isxdigit(c);
    if (!hex) return bail("revision must be a 7..=64 character hex commit ID");
    static const char* archs[] = {"sm_80", "sm_89", "sm_90", "sm_100", "sm_121"};
    bool arch_ok = false;
    for (const char* a : archs) arch_ok = arch_ok || m->arch == a;
    if (!arch_ok) return bail("unsupported kernel architecture " + m->arch);
    // 1..=MAX_ARTIFACTS entries (v3/crates/rvllm-kernels/src/manifest.rs:190-195)
    if (m->entries.empty() || m->entries.size() > MAX_ARTIFACTS) return bail("artifact count must be in 1..=4096");
    std::string dir = manifest_path;
    size_t slash = dir.rfind('/');
    dir = slash == std::string::npos ? "." : dir.substr(0, slash);
    // The manifest directory and every artifact are resolved (symlinks included) and the artifact must
    // still lie under the resolved directory, as manifest.rs:197-238 does with canonicalize/starts_with.
    char* root_c = realpath(dir.c_str(), nullptr);
    if (!root_c) return bail("cannot resolve the manifest directory");
    m->dir = root_c;
    free(root_c);
    uint64_t total_bytes = 0;
    for (auto& kv : m->entries) {
        Entry& e = kv.second;
        const std::string& name = kv.first;
        if (!name_ok(name, 128)) return bail("invalid artifact name " + name);
        if (!digest_ok(e.sha256)) return bail(name + ": sha256 must be 64 lowercase hex characters");
        if (!name_ok(e.abi, 64)) return bail(name + ": invalid ABI identifier");
        const bool agree = (e.kind == 0 && ends_with(e.path, ".ptx") && e.abi == "cuda-ptx-v1") ||
                           (e.kind == 1 && ends_with(e.path, ".so") && e.abi.rfind("rvllm-cuda-so-v", 0) == 0);
        if (!agree) return bail(name + ": artifact kind, extension, and ABI do not agree");
        if (!path_ok(e.path)) return bail(name + ": path must be relative and stay inside the manifest directory");
        if (e.bytes == 0 || e.bytes > MAX_ARTIFACT_BYTES) return bail(name + ": artifact size out of range");
        total_bytes += e.bytes;  // each term <= 512 MiB and at most 4096 terms: cannot overflow
        if (total_bytes > MAX_ARTIFACT_BYTES * 4) return bail("total artifact bytes exceed release limit");
        char* real_c = realpath((m->dir + "/" + e.path).c_str(), nullptr);
        if (!real_c) return bail(name + ": cannot resolve " + e.path);
        const std::string real = real_c;
        free(real_c);
        const std::string prefix = m->dir == "/" ? m->dir : m->dir + "/";
        if (real.compare(0, prefix.size(), prefix) != 0) return bail(name + ": artifact escapes manifest root");
        if (!read_bounded(real, MAX_ARTIFACT_BYTES, e.data, why)) return bail(name + ": " + why);
        if (e.data.size() != e.bytes) return bail(name + ": size differs from the manifest");
        if (sha256_hex(e.data.data(), e.data.size()) != e.sha256) return bail(name + ": sha256 differs from the manifest");
    }
    *out = m;
    return RVLLM_OK;
}

void rvllm_manifest_free(rvllm_manifest* m) { delete m; }
const char* rvllm_manifest_arch(const rvllm_manifest* m) { return m ? m->arch.c_str() : ""; }
const char* rvllm_manifest_revision(const rvllm_manifest* m) { return m ? m->revision.c_str() : ""; }
int rvllm_manifest_entry_count(const rvllm_manifest* m) { return m ? (int)m->entries.size() : -1; }

int rvllm_manifest_artifact(const rvllm_manifest* m, const char* name, const void** bytes, uint64_t* len, int* kind,
                            const char** abi) {
    if (!m || !name) return rv_fail(RVLLM_E_INVALID, "null argument");
    auto it = m->entries.find(name);
    if (it == m->entries.end()) return rv_fail(RVLLM_E_ARTIFACT, "artifact %s is not in the manifest", name);
    if (bytes) *bytes = it->second.data.data();
    if (len) *len = it->second.data.size();
    if (kind) *kind = it->second.kind;
    if (abi) *abi = it->second.abi.c_str();
    return RVLLM_OK;
}

}  // extern "C"

// ---- CUDA driver API, resolved at first use ---------------------------------------------------
namespace {

typedef int (*cuInit_t)(unsigned);
typedef int (*cuModuleLoadData_t)(void**, const void*);
typedef int (*cuModuleUnload_t)(void*);
typedef int (*cuModuleGetFunction_t)(void**, void*, const char*);
typedef int (*cuFuncSetAttribute_t)(void*, int, int);
typedef int (*cuLaunchKernel_t)(void*, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, void*,
                                void**, void**);
typedef int (*cuGetErrorString_t)(int, const char**);

struct Driver {
    void* lib = nullptr;
    cuInit_t init = nullptr;
    cuModuleLoadData_t load = nullptr;
    cuModuleUnload_t unload = nullptr;
    cuModuleGetFunction_t getfn = nullptr;
    cuFuncSetAttribute_t setattr = nullptr;
    cuLaunchKernel_t launch = nullptr;
    cuGetErrorString_t errstr = nullptr;
    bool ok = false;
};

Driver& driver() {
    static Driver d;
    static bool tried = false;
    if (!tried) {
        tried = true;
        d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (d.lib) {
            d.init = (cuInit_t)dlsym(d.lib, "cuInit");
            d.load = (cuModuleLoadData_t)dlsym(d.lib, "cuModuleLoadData");
            d.unload = (cuModuleUnload_t)dlsym(d.lib, "cuModuleUnload");
            d.getfn = (cuModuleGetFunction_t)dlsym(d.lib, "cuModuleGetFunction");
            d.setattr = (cuFuncSetAttribute_t)dlsym(d.lib, "cuFuncSetAttribute");
            d.launch = (cuLaunchKernel_t)dlsym(d.lib, "cuLaunchKernel");
            d.errstr = (cuGetErrorString_t)dlsym(d.lib, "cuGetErrorString");
            d.ok = d.init && d.load && d.unload && d.getfn && d.setattr && d.launch && d.init(0) == 0;
        }
    }
    return d;
}

int cu_fail(int code, const char* what) {
    const char* msg = nullptr;
    Driver& d = driver();
    if (d.errstr) d.errstr(code, &msg);
    return rv_fail(RVLLM_E_LAUNCH, "%s: CUDA driver error %d (%s)", what, code, msg ? msg : "?");
}

}  // namespace

struct rvllm_module {
    void* handle = nullptr;
    std::string name;
    std::vector<char> image;  // NUL-terminated PTX text
};

extern "C" {

int rvllm_module_load_ptx(rvllm_module** out, const rvllm_manifest* m, const char* name) {
    if (!out || !m || !name) return rv_fail(RVLLM_E_INVALID, "null argument");
    auto it = m->entries.find(name);
    if (it == m->entries.end()) return rv_fail(RVLLM_E_ARTIFACT, "artifact %s is not in the manifest", name);
    const Entry& e = it->second;
    if (e.kind != 0) return rv_fail(RVLLM_E_ARTIFACT, "artifact %s is not a PTX module", name);
    if (memchr(e.data.data(), 0, e.data.size())) return rv_fail(RVLLM_E_ARTIFACT, "PTX artifact %s has an interior NUL", name);
    Driver& d = driver();
    if (!d.ok) return rv_fail(RVLLM_E_NO_DEVICE, "CUDA driver is not available; PTX module %s cannot be loaded", name);
    rvllm_module* mod = new rvllm_module();
    mod->name = name;
    mod->image.assign((const char*)e.data.data(), (const char*)e.data.data() + e.data.size());
    mod->image.push_back('\0');
    int rc = d.load(&mod->handle, mod->image.data());
    if (rc != 0) {
        delete mod;
        return cu_fail(rc, "cuModuleLoadData");
    }
    *out = mod;
    return RVLLM_OK;
}

void rvllm_module_unload(rvllm_module* mod) {
    if (!mod) return;
    if (mod->handle && driver().ok) driver().unload(mod->handle);
    delete mod;
}

int rvllm_module_get_function(rvllm_module* mod, const char* symbol, void** function_out) {
    if (!mod || !symbol || !function_out) return rv_fail(RVLLM_E_INVALID, "null argument");
    int rc = driver().getfn(function_out, mod->handle, symbol);
    if (rc != 0) return rv_fail(RVLLM_E_ARTIFACT, "module %s has no entry point %s (driver error %d)", mod->name.c_str(), symbol, rc);
    return RVLLM_OK;
}

int rvllm_launch_raw(void* function, uint32_t grid_x, uint32_t grid_y, uint32_t grid_z, uint32_t block_x,
                     uint32_t block_y, uint32_t block_z, uint32_t dynamic_smem_bytes, void* stream, void** args) {
    if (!function) return rv_fail(RVLLM_E_INVALID, "null kernel function");
    if (!grid_x || !grid_y || !grid_z || !block_x || !block_y || !block_z) return rv_fail(RVLLM_E_INVALID, "zero launch dimension");
    if (grid_y > 65535 || grid_z > 65535 || grid_x > 2147483647u) return rv_fail(RVLLM_E_INVALID, "grid dimension too large");
    if ((uint64_t)block_x * block_y * block_z > 1024 || block_z > 64) return rv_fail(RVLLM_E_INVALID, "more than 1024 threads per block");
    if (dynamic_smem_bytes > 227 * 1024) return rv_fail(RVLLM_E_INVALID, "dynamic shared memory above the device limit");
    Driver& d = driver();
    if (!d.ok) return rv_fail(RVLLM_E_NO_DEVICE, "CUDA driver is not available");
    if (dynamic_smem_bytes > 48 * 1024) {
        int rc = d.setattr(function, 8 /* CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES */, (int)dynamic_smem_bytes);
        if (rc != 0) return cu_fail(rc, "cuFuncSetAttribute");
    }
    int rc = d.launch(function, grid_x, grid_y, grid_z, block_x, block_y, block_z, dynamic_smem_bytes, stream, args, nullptr);
    if (rc != 0) return cu_fail(rc, "cuLaunchKernel");
    return RVLLM_OK;
}

int rvllm_manifest_dlopen(const rvllm_manifest* m, const char* name, void** handle_out) {
    if (!m || !name || !handle_out) return rv_fail(RVLLM_E_INVALID, "null argument");
    auto it = m->entries.find(name);
    if (it == m->entries.end()) return rv_fail(RVLLM_E_ARTIFACT, "artifact %s is not in the manifest", name);
    const Entry& e = it->second;
    if (e.kind != 1) return rv_fail(RVLLM_E_ARTIFACT, "artifact %s is not a shared object", name);
    // the verified bytes go into a sealed memfd so that what is mapped is what was hashed
    int fd = memfd_create(name, MFD_CLOEXEC | MFD_ALLOW_SEALING);
    if (fd < 0) return rv_fail(RVLLM_E_ARTIFACT, "memfd_create failed for %s", name);
    size_t off = 0;
    while (off < e.data.size()) {
        ssize_t n = write(fd, e.data.data() + off, e.data.size() - off);
        if (n <= 0) {
            close(fd);
            return rv_fail(RVLLM_E_ARTIFACT, "short write into the sealed copy of %s", name);
        }
        off += (size_t)n;
    }
    if (fcntl(fd, F_ADD_SEALS, F_SEAL_SHRINK | F_SEAL_GROW | F_SEAL_WRITE | F_SEAL_SEAL) != 0) {
        close(fd);
        return rv_fail(RVLLM_E_ARTIFACT, "cannot seal the copy of %s", name);
    }
    char path[64];
    snprintf(path, sizeof path, "/proc/self/fd/%d", fd);
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    close(fd);
    if (!h) return rv_fail(RVLLM_E_ARTIFACT, "dlopen of %s failed: %s", name, dlerror());
    *handle_out = h;
    return RVLLM_OK;
}

}  // extern "C"
