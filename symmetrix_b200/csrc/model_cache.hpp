// Binary side-car of a parsed model file.
//
// A production-size model file is hundreds of megabytes of JSON text (the radial tables of a K = 128, 5-element model:
// 314 MB), and parsing it dominates start-up (3.3 s). After the first load the parsed and re-laid-out tables are written
// next to the file as `<file>.smxcache`; later loads read that instead. The side-car is tied to the exact source file
// (size and modification time) and to the build of this library (its format tag is the compilation time stamp), and it is
// only an accelerator: any mismatch, short read or write failure falls back to the JSON text. SMX_MODEL_CACHE=0 turns it off.
// The reference parses its JSON on every start (MACE::load_from_json, mace.cpp:905-1030).
#pragma once

#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "model.hpp"

namespace smx {

namespace detail {

// One description of the model's members, used for writing, reading and hashing.
template <class Ar>
void visit_program(Ar& ar, PolyProgram& p) {
    ar(p.words); ar(p.num_monomials); ar(p.num_leaves); ar(p.num_pairs); ar(p.alias);
}
template <class Ar>
void visit_programs(Ar& ar, std::vector<PolyProgram>& v) {
    int n = static_cast<int>(v.size());
    ar(n);
    v.resize(n);
    for (auto& p : v) visit_program(ar, p);
}
template <class Ar>
void visit_model(Ar& ar, HostModel& m) {
    ar(m.num_elements); ar(m.K); ar(m.l_max); ar(m.L_max); ar(m.num_lm); ar(m.num_LM); ar(m.r_cut);
    ar(m.atomic_numbers); ar(m.atomic_energies); ar(m.has_zbl);
    ar(m.zbl_a_exp); ar(m.zbl_a_prefactor); ar(m.zbl_c); ar(m.zbl_covalent_radii); ar(m.zbl_p);
    ar(m.A0_scaled); ar(m.A1_scaled); ar(m.A0_spline_h); ar(m.A1_spline_h); ar(m.A0_spline_bins); ar(m.A1_spline_bins);
    ar(m.A0_spline_coef); ar(m.A1_spline_coef);
    ar(m.spline_h); ar(m.num_bins); ar(m.num_pairs); ar(m.F0); ar(m.F1); ar(m.coef0); ar(m.coef1);
    ar(m.H0_w); ar(m.A0_w); ar(m.H1_w); ar(m.A1_w);
    for (auto& o : m.A1_w_off) ar(o);
    ar(m.H2_w_H1); ar(m.H2_w_M1); ar(m.ro1); ar(m.ro2_w1); ar(m.ro2_w2); ar(m.ro2_scale);
    ar(m.path_file_to_canon); ar(m.lme_file_to_canon); ar(m.path_scale);
    ar(m.rmlp1.present); ar(m.rmlp1.num_bessel); ar(m.rmlp1.poly_p); ar(m.rmlp1.hidden); ar(m.rmlp1.num_hidden_layers);
    ar(m.rmlp1.silu_scale); ar(m.rmlp1.w_first); ar(m.rmlp1.w_hidden); ar(m.rmlp1.w_last); ar(m.rmlp1.pair_scale); ar(m.rmlp1.basis_coef);
    visit_programs(ar, m.prog0); ar(m.mono_off0); ar(m.num_mono0); ar(m.coef_M0);
    visit_program(ar, m.prog1); ar(m.num_mono1); ar(m.coef_M1);
    ar(m.poly_canonical); ar(m.num_canon0); ar(m.num_canon1); ar(m.coef_M0_canon); ar(m.coef_M1_canon);
    ar(m.num_interactions); ar(m.coefm); ar(m.Am_w);
    for (auto& o : m.Am_w_off) ar(o);
    visit_programs(ar, m.progm); ar(m.mono_offm); ar(m.num_monom); ar(m.num_canonm); ar(m.coef_Mm); ar(m.coef_Mm_canon);
    ar(m.Hm_w); ar(m.Hm_res); ar(m.ro_m);
}

struct Writer {
    FILE* f; bool ok = true;
    void raw(const void* p, size_t n) { if (ok && n && std::fwrite(p, 1, n, f) != n) ok = false; }
    template <typename T> void pod(const T& v) { raw(&v, sizeof(T)); }
    void operator()(int& v) { pod(v); }
    void operator()(long& v) { pod(v); }
    void operator()(double& v) { pod(v); }
    void operator()(bool& v) { const int b = v ? 1 : 0; pod(b); }
    template <typename T> void operator()(std::vector<T>& v) { const uint64_t n = v.size(); pod(n); raw(v.data(), n * sizeof(T)); }
};
struct Reader {
    FILE* f; bool ok = true;
    void raw(void* p, size_t n) { if (ok && n && std::fread(p, 1, n, f) != n) ok = false; }
    template <typename T> void pod(T& v) { raw(&v, sizeof(T)); }
    void operator()(int& v) { pod(v); }
    void operator()(long& v) { pod(v); }
    void operator()(double& v) { pod(v); }
    void operator()(bool& v) { int b = 0; pod(b); v = b != 0; }
    template <typename T> void operator()(std::vector<T>& v) {
        uint64_t n = 0; pod(n);
        if (!ok || n > (1ull << 34)) { ok = false; return; }
        v.resize(n); raw(v.data(), n * sizeof(T));
    }
};
struct Hasher {     // FNV-1a over the same byte stream the writer produces
    uint64_t h = 1469598103934665603ull;
    void raw(const void* p, size_t n) { const unsigned char* c = static_cast<const unsigned char*>(p); for (size_t i = 0; i < n; ++i) { h ^= c[i]; h *= 1099511628211ull; } }
    template <typename T> void pod(const T& v) { raw(&v, sizeof(T)); }
    void operator()(int& v) { pod(v); }
    void operator()(long& v) { pod(v); }
    void operator()(double& v) { pod(v); }
    void operator()(bool& v) { const int b = v ? 1 : 0; pod(b); }
    template <typename T> void operator()(std::vector<T>& v) { const uint64_t n = v.size(); pod(n); raw(v.data(), n * sizeof(T)); }
};

struct CacheHeader {
    char magic[8];          // "SMXCACHE"
    char build[32];         // compilation time stamp of the library: a rebuilt library never reads an older layout
    int64_t source_size, source_mtime_ns;
};
inline CacheHeader make_header(const struct stat& st) {
    CacheHeader h{};
    std::memcpy(h.magic, "SMXCACHE", 8);
    std::snprintf(h.build, sizeof(h.build), "%s %s", __DATE__, __TIME__);
    h.source_size = static_cast<int64_t>(st.st_size);
    h.source_mtime_ns = static_cast<int64_t>(st.st_mtim.tv_sec) * 1000000000ll + st.st_mtim.tv_nsec;
    return h;
}

}  // namespace detail

inline uint64_t model_digest(HostModel& m) {
    detail::Hasher h;
    detail::visit_model(h, m);
    return h.h;
}

// Loads through the side-car when it is valid, else parses the JSON text and (best effort) writes the side-car.
// `used_cache` (optional) reports which of the two happened.
inline HostModel load_model_cached(const std::string& filename, bool* used_cache = nullptr) {
    if (used_cache) *used_cache = false;
    const char* env = std::getenv("SMX_MODEL_CACHE");
    struct stat st{};
    const bool enabled = !(env && std::string(env) == "0") && stat(filename.c_str(), &st) == 0;
    if (!enabled) return load_model_file(filename);
    const std::string side = filename + ".smxcache";
    const detail::CacheHeader want = detail::make_header(st);
    if (FILE* f = std::fopen(side.c_str(), "rb")) {
        detail::CacheHeader got{};
        HostModel m;
        detail::Reader rd{f};
        rd.raw(&got, sizeof(got));
        if (rd.ok && std::memcmp(&got, &want, sizeof(got)) == 0) {
            detail::visit_model(rd, m);
            char tail = 0;
            const bool at_end = std::fread(&tail, 1, 1, f) == 0;
            std::fclose(f);
            if (rd.ok && at_end) {
                m.tp = make_tp_table(m.L_max);
                if (used_cache) *used_cache = true;
                return m;
            }
        } else {
            std::fclose(f);
        }
    }
    HostModel m = load_model_file(filename);
    const std::string tmp = side + ".tmp" + std::to_string(static_cast<long>(getpid()));
    if (FILE* f = std::fopen(tmp.c_str(), "wb")) {
        detail::Writer wr{f};
        wr.raw(&want, sizeof(want));
        detail::visit_model(wr, m);
        const bool ok = wr.ok && std::fclose(f) == 0;
        if (!ok || std::rename(tmp.c_str(), side.c_str()) != 0) std::remove(tmp.c_str());
    }
    return m;
}

}  // namespace smx
