// A stand-in for the two decomposed compute() modes of the reference's LAMMPS pair style, compiled against the C++ facade
// (include/symmetrix_b200_mace.hpp) and run for all ranks of a slab decomposition inside one process:
//   mode 0  PairSymmetrixMACE::compute_mpi_message_passing      (pair_symmetrix/pair_symmetrix_mace.cpp:376-547)
//   mode 1  PairSymmetrixMACE::compute_no_mpi_message_passing   (pair_symmetrix/pair_symmetrix_mace.cpp:551-748)
// The stage calls carry the reference's argument lists and come in the reference's order; the only additions are
// begin() where the pair style zero-fills node_energies / node_forces, and pull() / push() around the halo exchanges where
// it reads or assigns mace->H1 / mace->H1_adj. LAMMPS' Comm (forward_comm / reverse_comm) is played by loops over the
// ranks' host vectors with the send / receive row lists the test wrote.
// Usage: pair_harness model.json mode num_ranks case_prefix out_prefix   (files <prefix><rank>.bin)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
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

struct Peer {
    int rank;
    std::vector<int> send_rows, recv_rows;   // my owned rows the peer has as ghosts (in its order); my ghost rows owned by the peer
};

struct Rank {
    int nlocal = 0, nall = 0, num_recv = 0;    // owned atoms, owned + ghost atoms, receivers in the arrays
    std::vector<int> node_types, num_neigh, neigh_indices, neigh_types;
    std::vector<double> xyz, r;
    std::vector<Peer> peers;
    std::unique_ptr<symmetrix_b200::MACE> mace;
    std::vector<double> H1, H1_adj, f;         // the pair style's own vectors (rows of all local + ghost atoms)
    double eng = 0.0;
};

static Rank read_rank(const std::string& path, const char* model) {
    Rank rk;
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); std::exit(3); }
    auto head = read_vec<int>(f);
    rk.nlocal = head[0]; rk.nall = head[1]; rk.num_recv = head[2];
    rk.node_types = read_vec<int>(f); rk.num_neigh = read_vec<int>(f);
    rk.neigh_indices = read_vec<int>(f); rk.neigh_types = read_vec<int>(f);
    rk.xyz = read_vec<double>(f); rk.r = read_vec<double>(f);
    const int npeers = head[3];
    for (int q = 0; q < npeers; ++q) {
        Peer p;
        p.rank = read_vec<int>(f)[0];
        p.send_rows = read_vec<int>(f);
        p.recv_rows = read_vec<int>(f);
        rk.peers.push_back(std::move(p));
    }
    std::fclose(f);
    rk.mace = std::make_unique<symmetrix_b200::MACE>(model);
    return rk;
}

static const Peer& peer_of(const Rank& rk, int rank) {
    for (const Peer& p : rk.peers) if (p.rank == rank) return p;
    std::abort();
}

// f[i] -= nf_ij, f[j] += nf_ij over the receivers evaluated (pair_symmetrix_mace.cpp:516-530, 716-731) and the energy sum
static void accumulate_forces(Rank& rk, int num_nodes, int num_energy_nodes) {
    auto& mace = *rk.mace;
    mace.pull("node_energies"); mace.pull("node_forces");
    rk.eng = 0.0;
    for (int ii = 0; ii < num_energy_nodes; ++ii) rk.eng += mace.node_energies[ii];
    rk.f.assign(3 * static_cast<size_t>(rk.nall), 0.0);
    long ij = 0;
    for (int ii = 0; ii < num_nodes; ++ii)
        for (int jj = 0; jj < rk.num_neigh[ii]; ++jj) {
            const int j = rk.neigh_indices[ij];
            for (int c = 0; c < 3; ++c) {
                rk.f[3 * ii + c] -= mace.node_forces[3 * ij + c];
                rk.f[3 * j + c] += mace.node_forces[3 * ij + c];
            }
            ij += 1;
        }
}

int main(int argc, char** argv) {
    if (argc != 6) return 2;
    try {
        const int mode = std::atoi(argv[2]), world = std::atoi(argv[3]);
        std::vector<Rank> ranks;
        for (int q = 0; q < world; ++q) ranks.push_back(read_rank(std::string(argv[4]) + std::to_string(q) + ".bin", argv[1]));
        const size_t width = static_cast<size_t>(ranks[0].mace->num_LM) * ranks[0].mace->num_channels;

        if (mode == 0) {
            // ---- compute_mpi_message_passing: receivers are the owned atoms
            for (Rank& rk : ranks) {
                auto& mace = *rk.mace;
                const int num_nodes = rk.nlocal;
                mace.begin(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_indices, rk.neigh_types, rk.xyz, rk.r);
                if (mace.has_zbl)
                    mace.zbl.compute_ZBL(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, mace.atomic_numbers, rk.r, rk.xyz,
                                         mace.node_energies, mace.node_forces);
                mace.compute_Y(rk.xyz);
                mace.compute_R0(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_A0(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types);
                mace.compute_A0_scaled(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_M0(num_nodes, rk.node_types);
                mace.compute_H1(num_nodes);
                // "sort local H1 contributions by i": rows of all local + ghost atoms, owned rows filled (:463-469)
                rk.H1.assign(static_cast<size_t>(rk.nall) * width, 0.0);
                const auto& h = mace.pull("H1");
                std::copy(h.begin(), h.begin() + static_cast<size_t>(num_nodes) * width, rk.H1.begin());
            }
            // comm->forward_comm(this): owners' rows into the ghost rows (pack_forward_comm / unpack_forward_comm, :194-216)
            for (Rank& rk : ranks)
                for (const Peer& p : rk.peers) {
                    const Peer& back = peer_of(ranks[p.rank], static_cast<int>(&rk - ranks.data()));
                    for (size_t m = 0; m < p.send_rows.size(); ++m)
                        std::copy(rk.H1.begin() + p.send_rows[m] * width, rk.H1.begin() + (p.send_rows[m] + 1) * width,
                                  ranks[p.rank].H1.begin() + back.recv_rows[m] * width);
                }
            for (Rank& rk : ranks) {
                auto& mace = *rk.mace;
                const int num_nodes = rk.nlocal;
                mace.H1 = rk.H1;                  // mace->H1 = H1 (:471)
                mace.push("H1");
                mace.compute_R1(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_Phi1(num_nodes, rk.num_neigh, rk.neigh_indices);
                mace.compute_A1(num_nodes);
                mace.compute_A1_scaled(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_M1(num_nodes, rk.node_types);
                mace.compute_H2(num_nodes, rk.node_types);
                mace.compute_readouts(num_nodes, rk.node_types);
                mace.reverse_H2(num_nodes, rk.node_types, false);
                mace.reverse_M1(num_nodes, rk.node_types);
                mace.reverse_A1_scaled(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r, false);
                mace.reverse_A1(num_nodes);
                mace.reverse_Phi1(num_nodes, rk.num_neigh, rk.neigh_indices, rk.xyz, rk.r, false, false);
                rk.H1_adj = mace.pull("H1_adj");  // H1_adj = mace->H1_adj (:488)
            }
            // comm->reverse_comm(this): ghost rows added into the owners' rows (pack_reverse_comm / unpack_reverse_comm, :218-238)
            for (Rank& rk : ranks)
                for (const Peer& p : rk.peers) {
                    const Peer& back = peer_of(ranks[p.rank], static_cast<int>(&rk - ranks.data()));
                    for (size_t m = 0; m < p.recv_rows.size(); ++m)
                        for (size_t k = 0; k < width; ++k)
                            ranks[p.rank].H1_adj[back.send_rows[m] * width + k] += rk.H1_adj[p.recv_rows[m] * width + k];
                }
            for (Rank& rk : ranks) {
                auto& mace = *rk.mace;
                const int num_nodes = rk.nlocal;
                mace.H1_adj = rk.H1_adj;          // mace->H1_adj = H1_adj (:490)
                mace.push("H1_adj");
                mace.reverse_H1(num_nodes);
                mace.reverse_M0(num_nodes, rk.node_types);
                mace.reverse_A0_scaled(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r);
                mace.reverse_A0(num_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r);
                accumulate_forces(rk, num_nodes, num_nodes);
            }
        } else {
            // ---- compute_no_mpi_message_passing: layer 0 on owned atoms + ghosts within r_cut, layer 1 on owned atoms
            for (Rank& rk : ranks) {
                auto& mace = *rk.mace;
                const int num_local_nodes = rk.nlocal, num_ghost_nodes = rk.num_recv - rk.nlocal;
                mace.begin(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_indices, rk.neigh_types, rk.xyz, rk.r);
                if (mace.has_zbl)
                    mace.zbl.compute_ZBL(num_local_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, mace.atomic_numbers, rk.r, rk.xyz,
                                         mace.node_energies, mace.node_forces);
                mace.compute_Y(rk.xyz);
                mace.compute_R0(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_A0(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_types);
                mace.compute_A0_scaled(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_M0(num_local_nodes + num_ghost_nodes, rk.node_types);
                mace.compute_H1(num_local_nodes + num_ghost_nodes);
                mace.compute_R1(num_local_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_Phi1(num_local_nodes, rk.num_neigh, rk.neigh_indices);
                mace.compute_A1(num_local_nodes);
                mace.compute_A1_scaled(num_local_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.r);
                mace.compute_M1(num_local_nodes, rk.node_types);
                mace.compute_H2(num_local_nodes, rk.node_types);
                mace.compute_readouts(num_local_nodes, rk.node_types);
                mace.reverse_H2(num_local_nodes, rk.node_types, false);
                mace.reverse_M1(num_local_nodes, rk.node_types);
                mace.reverse_A1_scaled(num_local_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r, false);
                mace.reverse_A1(num_local_nodes);
                mace.reverse_Phi1(num_local_nodes, rk.num_neigh, rk.neigh_indices, rk.xyz, rk.r, false, false);
                mace.reverse_H1(num_local_nodes + num_ghost_nodes);
                mace.reverse_M0(num_local_nodes + num_ghost_nodes, rk.node_types);
                mace.reverse_A0_scaled(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r);
                mace.reverse_A0(num_local_nodes + num_ghost_nodes, rk.node_types, rk.num_neigh, rk.neigh_types, rk.xyz, rk.r);
                accumulate_forces(rk, num_local_nodes + num_ghost_nodes, num_local_nodes);
            }
        }
        // LAMMPS adds the forces on ghost atoms to their owners after the pair style returns (reverse communication of f)
        std::vector<std::vector<double>> owned(world);
        for (int q = 0; q < world; ++q) owned[q].assign(ranks[q].f.begin(), ranks[q].f.begin() + 3 * static_cast<size_t>(ranks[q].nlocal));
        for (int q = 0; q < world; ++q)
            for (const Peer& p : ranks[q].peers) {
                const Peer& back = peer_of(ranks[p.rank], q);
                for (size_t m = 0; m < p.recv_rows.size(); ++m)
                    for (int c = 0; c < 3; ++c) owned[p.rank][3 * back.send_rows[m] + c] += ranks[q].f[3 * p.recv_rows[m] + c];
            }
        for (int q = 0; q < world; ++q) {
            FILE* o = std::fopen((std::string(argv[5]) + std::to_string(q) + ".bin").c_str(), "wb");
            std::fwrite(&ranks[q].eng, sizeof(double), 1, o);
            std::fwrite(owned[q].data(), sizeof(double), owned[q].size(), o);
            std::fclose(o);
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "pair_harness: %s\n", e.what());
        return 1;
    }
    return 0;
}
