"""Worker of the multi-GPU decomposition test: launched with torch.distributed.run, one rank per GPU.
Evaluates a decomposed structure over NCCL and compares with the single-domain evaluation on rank 0's GPU."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from symmetrix_b200 import MACE, structures as st  # noqa: E402
from symmetrix_b200.domain import SlabRank, evaluate_decomposed, make_slab_plan  # noqa: E402


def main():
    model, dtype, out = sys.argv[1], sys.argv[2], sys.argv[3]
    mode = sys.argv[4] if len(sys.argv) > 4 else "message_passing"
    transport = sys.argv[5] if len(sys.argv) > 5 else "torch"      # "library": NCCL send / recv issued inside libsymmetrix_b200
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ev = MACE(model, dtype=dtype, device=local)
    if transport == "library":
        ev.comm_init(dist)
    s = st.fcc_box((4 * world, 3, 3), 3.6, ev.atomic_numbers, seed=17, jitter=0.12)
    rk = SlabRank(make_slab_plan(s, ev.r_cut, rank, world, mode=mode), ev, ev.r_cut, ev.atomic_numbers)
    rk.build_edges()
    for _ in range(2):
        energy, virial, owned = evaluate_decomposed([rk], dist=dist)
    gathered = [None] * world
    dist.all_gather_object(gathered, (rk.plan.own_global, owned[0].cpu().numpy()))
    if rank == 0:
        forces = np.zeros((s.num_atoms, 3))
        for own, f in gathered:
            forces[own] = f
        single = MACE(model, dtype="float64", device=local)
        nl = st.neighbor_list(s, single.r_cut)
        inp = st.evaluator_inputs(s, nl, single.atomic_numbers)
        single.compute_node_energies_forces(inp["num_nodes"], inp["node_types"], inp["num_neigh"], inp["neigh_indices"],
                                            inp["neigh_types"], inp["xyz"], inp["r"])
        f_ref, v_ref, e_ref = single.reduce_forces()
        np.savez(out, energy=energy, e_ref=e_ref, forces=forces, f_ref=f_ref, virial=virial, v_ref=v_ref)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
