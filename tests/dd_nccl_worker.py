"""Worker of test_gpu_domain_nccl.py: one rank of a 2-GPU NCCL run; rank 0 writes energy and forces to the given file."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(out):
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from so3lr_b200 import domain as D
    from so3lr_b200 import workloads as W
    Z, R, cell = W.water_box(1000, 31.0, 21, jitter=0.02)
    V, m = W.maxwell_boltzmann(Z, 300.0, 22)
    be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=0.5, device=local)
    dom = D.DomainSystem(D.DistComm(), be, Z, R, cell, skin=0.5, cutoff_lr=12.0, velocities=V, masses=m, device=dev)
    E0, _ = dom.compute(check_rebuild=False)
    F0 = dom.global_forces().cpu().numpy()
    dom.nve(20, 0.5)
    R1 = dom.gather_global(dom.R[: dom.n0]).cpu().numpy()
    F1 = dom.global_forces().cpu().numpy()
    E1 = float(dom.E)
    # the same positions with the reciprocal-space sum on: the charge mesh is all-reduced over NCCL
    dom.set_kspace((32, 32, 32), 2.0, "pme")
    Ek, _ = dom.compute(check_rebuild=False)
    Fk = dom.global_forces().cpu().numpy()
    if rank == 0:
        np.savez(out, E0=float(E0), F0=F0, R1=R1, F1=F1, E1=E1, rebuilds=dom.n_rebuilds, Ek=float(Ek), Fk=Fk)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
