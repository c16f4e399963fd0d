// Compiles the C++ facade and replays, against it, the single-domain compute() of the reference's
// LAMMPS pair style (pair_symmetrix/pair_symmetrix_mace.cpp:242-372) on arrays read from a small
// binary file written by the test: edge filter -> CSR -> evaluation -> f[i] -= nf, f[j] += nf.
// Usage: facade_harness model.json case.bin out.bin
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "symmetrix_b200_mace.hpp"

template <typename T>
static std::vector<T> read_vec(FILE* f) {
    long n = 0;
    if (std::fread(&n, sizeof(long), 1, f) != 1) std::abort();
    std::vector<T> v(n);
    if (n && std::fread(v.data(), sizeof(T), n, f) != static_cast<size_t>(n)) std::abort();
    return v;
}

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    try {
        symmetrix_b200::MACE mace(argv[1]);
        FILE* f = std::fopen(argv[2], "rb");
        if (!f) return 3;
        auto node_types = read_vec<int>(f);
        auto num_neigh = read_vec<int>(f);
        auto neigh_indices = read_vec<int>(f);
        auto neigh_types = read_vec<int>(f);
        auto xyz = read_vec<double>(f);
        auto r = read_vec<double>(f);
        std::fclose(f);
        const int num_nodes = static_cast<int>(node_types.size());
        mace.compute_node_energies_forces(num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r);
        double eng = 0.0;
        for (int ii = 0; ii < num_nodes; ++ii) eng += mace.node_energies[ii];
        std::vector<double> force(3 * num_nodes, 0.0);
        long ij = 0;
        for (int ii = 0; ii < num_nodes; ++ii)
            for (int jj = 0; jj < num_neigh[ii]; ++jj) {
                const int j = neigh_indices[ij];
                for (int c = 0; c < 3; ++c) {
                    force[3 * ii + c] -= mace.node_forces[3 * ij + c];
                    force[3 * j + c] += mace.node_forces[3 * ij + c];
                }
                ij += 1;
            }
        // the same reduction done by the library
        std::vector<double> force2(3 * num_nodes, 0.0);
        double virial[6], eng2 = 0.0;
        mace.reduce_forces(num_nodes, force2.data(), virial, &eng2);
        FILE* o = std::fopen(argv[3], "wb");
        std::fwrite(&eng, sizeof(double), 1, o);
        std::fwrite(&eng2, sizeof(double), 1, o);
        std::fwrite(force.data(), sizeof(double), force.size(), o);
        std::fwrite(force2.data(), sizeof(double), force2.size(), o);
        std::fclose(o);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "facade_harness: %s\n", e.what());
        return 1;
    }
    return 0;
}
