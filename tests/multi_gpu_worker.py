"""Worker of tests/test_gpu_multi.py: one rank of a deterministic sharded run through the library's own
multi-GPU path (mascot_shard_*: C++ schedule, NCCL hand-overs).  Started as a plain process per rank;
the 128-byte group id travels through a file.  Writes this rank's results for the parent test.

    python multi_gpu_worker.py <out_dir> <rank> <world> <blocks_per_gpu>
"""
import importlib.util
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
from test_multi_cpu import HYPER, dataset  # noqa: E402


def main():
    out_dir, rank, world, per_gpu = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    spec = importlib.util.spec_from_file_location("mascot_binding", os.path.join(ROOT, "icdm-2021_mascot_b200", "mascot.py"))
    M = importlib.util.module_from_spec(spec); sys.modules["mascot_binding"] = M; spec.loader.exec_module(M)
    id_path = os.path.join(out_dir, "group.id")
    if rank == 0:
        with open(id_path + ".tmp", "wb") as f:
            f.write(M.comm_unique_id())
        os.replace(id_path + ".tmp", id_path)
    deadline = time.time() + 120
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise SystemExit("no group id within two minutes")
        time.sleep(0.05)
    comm_id = open(id_path, "rb").read()
    R, test, P, Q, n_users, n_items = dataset()
    cfg = M.default_config(version=M.V_MASCOT, k=HYPER["k"], deterministic=1, shuffle=0, epoch=HYPER["epochs"],
                           learning_rate=HYPER["lr"], decay=HYPER["decay"], lam=HYPER["lam"], user_group_num=HYPER["ug"],
                           item_group_num=HYPER["ig"], sample_ratio=HYPER["sample_ratio"], interval=HYPER["interval"],
                           error_threshold=HYPER["threshold"], device=rank)
    eng = M.Engine(cfg)
    eng.shard_init(comm_id, rank, world, per_gpu, timeout_ms=60000)
    eng.shard_set_ratings(R, test, n_users, n_items)
    eng.set_factors(P, Q)
    rm, promoted = [], []
    for e in range(8):
        st = eng.shard_train_epoch(e)
        rm.append(eng.shard_eval_rmse())
        promoted.append([st.promoted_user_groups, st.promoted_item_groups])
    info = eng.shard_info()
    eng.shard_gather_factors()
    Pm, Qm = eng.get_factors(1)
    uprec, iprec = eng.group_info(0)[1], eng.group_info(1)[1]
    u2s, i2s = eng.index_maps()
    np.savez(os.path.join(out_dir, f"gpu_rank{rank}.npz"), P=Pm, Q=Qm, rmse=np.array(rm), promoted=np.array(promoted),
             uprec=uprec, iprec=iprec, u2s=u2s, i2s=i2s, local=info["local_ratings"], sent=info["bytes_sent"],
             test_ratings=eng.test_ratings(1))
    eng.close()


if __name__ == "__main__":
    main()
