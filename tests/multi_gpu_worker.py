"""Worker of tests/test_gpu_multi.py: one rank of a 2-GPU deterministic sharded run.  Launched with
torch.distributed.run; writes this rank's factors for the parent test to compare with the replay."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
from test_multi_cpu import HYPER, dataset, load_multi  # noqa: E402


def main():
    import importlib.util
    out_dir = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    spec = importlib.util.spec_from_file_location("mascot_binding", os.path.join(ROOT, "icdm-2021_mascot_b200", "mascot.py"))
    M = importlib.util.module_from_spec(spec); sys.modules["mascot_binding"] = M; spec.loader.exec_module(M)
    multi = load_multi()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    try:
        R, test, P, Q, n_users, n_items = dataset()
        plan = multi.make_plan(R["u"], R["i"], n_users, n_items, world)
        cfg = M.default_config(version=M.V_MASCOT, k=HYPER["k"], deterministic=1, shuffle=0, epoch=HYPER["epochs"],
                               learning_rate=HYPER["lr"], decay=HYPER["decay"], lam=HYPER["lam"], user_group_num=HYPER["ug"],
                               item_group_num=HYPER["ig"], sample_ratio=HYPER["sample_ratio"], interval=HYPER["interval"],
                               error_threshold=HYPER["threshold"], device=local)
        shard = multi.EngineShard(M, cfg, plan, rank, R, test, n_users, n_items)
        shard.engine.set_factors(P, Q)
        rm, promoted = [], []
        for e in range(8):
            _, pr = multi.train_epoch(dist, shard, rank, world, e, comm_device=dev)
            multi.gather_item_factors(dist, shard, world)
            rm.append(multi.global_rmse(dist, shard, world, comm_device=dev))
            promoted.append(pr)
        Pm, Qm = shard.engine.get_factors(1)
        uprec, iprec = shard.engine.group_info(0)[1], shard.engine.group_info(1)[1]
        np.savez(os.path.join(out_dir, f"gpu_rank{rank}.npz"), P=Pm, Q=Qm, rmse=np.array(rm), promoted=np.array(promoted),
                 uprec=uprec, iprec=iprec)
        shard.close()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
