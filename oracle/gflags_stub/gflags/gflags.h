// Minimal stand-in for <gflags/gflags.h>, enough to build the SpTMM reference's main.cu
// (gflags itself is not installed here).  TEST INFRASTRUCTURE ONLY: used by ref_harness.cu.
// Accepts -flag value, -flag=value, --flag=value; booleans also as bare -flag / -noflag.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <cstdio>

namespace gflags_stub {
struct Flag { const char *name; char kind; void *ptr; };
inline std::vector<Flag> &registry() { static std::vector<Flag> r; return r; }
struct Registrar { Registrar(const char *n, char k, void *p) { registry().push_back({n, k, p}); } };
inline bool assign(const Flag &f, const char *v) {
    switch (f.kind) {
        case 'b': *(bool *)f.ptr = !(strcmp(v, "false") == 0 || strcmp(v, "0") == 0); return true;
        case 'q': *(uint64_t *)f.ptr = strtoull(v, nullptr, 10); return true;
        case 'u': *(uint32_t *)f.ptr = (uint32_t)strtoul(v, nullptr, 10); return true;
    }
    return false;
}
}  // namespace gflags_stub

#define DEFINE_bool(name, val, txt)   bool FLAGS_##name = val; \
    static gflags_stub::Registrar reg_##name(#name, 'b', &FLAGS_##name)
#define DEFINE_uint64(name, val, txt) uint64_t FLAGS_##name = val; \
    static gflags_stub::Registrar reg_##name(#name, 'q', &FLAGS_##name)
#define DEFINE_uint32(name, val, txt) uint32_t FLAGS_##name = val; \
    static gflags_stub::Registrar reg_##name(#name, 'u', &FLAGS_##name)

namespace gflags {
inline void SetUsageMessage(const std::string &) {}
inline uint32_t ParseCommandLineFlags(int *argc, char ***argv, bool) {
    using namespace gflags_stub;
    for (int i = 1; i < *argc; i++) {
        const char *a = (*argv)[i];
        if (a[0] != '-') continue;
        while (*a == '-') a++;
        std::string key(a), val;
        bool has_val = false;
        size_t eq = key.find('=');
        if (eq != std::string::npos) { val = key.substr(eq + 1); key = key.substr(0, eq); has_val = true; }
        bool found = false;
        for (const Flag &f : registry()) {
            if (key == f.name) {
                if (f.kind == 'b' && !has_val) { *(bool *)f.ptr = true; }
                else {
                    if (!has_val && i + 1 < *argc) { val = (*argv)[++i]; }
                    assign(f, val.c_str());
                }
                found = true; break;
            }
            if (f.kind == 'b' && key == std::string("no") + f.name) { *(bool *)f.ptr = false; found = true; break; }
        }
        if (!found) { fprintf(stderr, "ERROR: unknown command line flag '%s'\n", key.c_str()); exit(1); }
    }
    return 1;
}
}  // namespace gflags
