"""GPU ranks for the sharded path (run by test_sharded_gpu.py; one process per GPU, NCCL).
Each rank's slice of the global batch -- indices and gathered bytes -- must equal the oracle's
single-process gather from the concatenated table."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from gear_b200 import _native as N  # noqa: E402
from gear_b200 import core  # noqa: E402
from gear_b200.comm import Communicator  # noqa: E402
from gear_b200.sharded import ShardedReplay  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    rank = int(os.environ.get("RANK", "0")); W = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    core.init(local)
    dev = torch.device("cuda", local)
    comm = None
    if W > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator.from_torch_distributed()
    rows, T, cap, L = [4096, 4, 12, 1], 64, 128, 16     # 8192 steps per shard
    n_local = cap * T
    b = 96
    B = b * W
    cols = list(range(len(rows)))

    def shard_data(r):
        accu, stride = O.table_layout(rows, T)
        img = O.philox_u32(100 + r, 0, 0, (stride * cap + 3) // 4).view(np.uint8)[: stride * cap].copy()
        prio = O.synth_lognormal(200 + r, 0, n_local)
        prio[r::5] = 0.0
        return img, prio

    img, prio = shard_data(rank)
    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM); table.connect(); table.write(0, img)
    handler = core.StorageHandler(table)
    handler.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    sampler = core.PrioritySampler(n_local)
    replay = ShardedReplay(handler, sampler, cols, rank, W, comm, max_global_batch=B)
    pbuf = core.DeviceBuffer(n_local * 4)        # an allocation of its own: the peers map it in the lazy pull mode
    dprio = pbuf.view(torch.float32)
    dprio.copy_(torch.from_numpy(prio))

    imgs, prios = zip(*[shard_data(r) for r in range(W)])
    gimg, gprio = np.concatenate(imgs), np.concatenate(prios)
    gcdf, gl1, _, _ = O.scan(gprio)
    accu, stride = O.table_layout(rows, T)
    def my_slice(x, layout):
        return x[rank * b:(rank + 1) * b] if layout == "contiguous" else x[rank::W]

    lazy_replay = ShardedReplay(handler, sampler, cols, rank, W, comm, max_global_batch=B, store=False)
    for trial in range(6):
        u01 = np.sort(O.synth_u01(300 + trial, 0, B))
        layout = "scattered" if trial >= 3 else "contiguous"
        if trial in (2, 5):
            u01[:] = np.sort(O.synth_u01(400, 0, B) * 0.01)     # every request lands on shard 0
        if trial == 0:      # routed request by request on the host
            outs, gflat = replay.step(dprio, u01)
        else:               # the device-resident route: same result by construction; 4, 5: tables without level 2
            rp = lazy_replay if trial >= 4 else replay
            outs, gflat = rp.step_sorted(dprio, u01, torch.from_numpy(u01).to(dev), layout=layout)
        torch.cuda.synchronize()
        want_flat = my_slice(O.search(gcdf, gl1, u01, scale=True), layout)
        assert np.array_equal(gflat.cpu().numpy(), want_flat), (rank, trial)
        gi, gt, gl = O.decode(want_flat, T)
        for c in cols:
            want = O.fused_subcopy(gimg, gi, gt, gl, stride, int(accu[c]), T, rows[c], 0, L, False)
            assert np.array_equal(outs[c].cpu().numpy(), want), (rank, trial, c)

    # exchange-free mode: the requester reads the owners' memory in place
    small = core.StorageHandler(table)                       # short segments: the staged copy path
    small.set(cols, [core.SubscribePattern(-1, 3, N.PAD_HEAD)] * len(rows))
    for mode, (double_buffer, ring, hd, off, Lm, head, lazy) in enumerate(
            [(True, False, handler, 0, L, False, False), (False, True, handler, 0, L, False, False),
             (True, False, small, -1, 3, True, False),
             (True, True, handler, 0, L, False, True), (True, False, small, -1, 3, True, True)]):
        rp = ShardedReplay(hd, sampler, cols, rank, W, comm, max_global_batch=B)
        rp.enable_pull(double_buffer=double_buffer, ring=ring, priorities=pbuf if lazy else None)
        for trial in range(6):
            u01 = np.sort(O.synth_u01(500 + trial, mode, B))
            layout = "scattered" if trial >= 4 else "contiguous"
            if trial == 2:
                u01[:] = np.sort(O.synth_u01(600, mode, B) * 0.01)
            outs, gflat = rp.step_pull(dprio, torch.from_numpy(u01).to(dev), rescan=(trial != 3), layout=layout)
            torch.cuda.synchronize()
            want_flat = my_slice(O.search(gcdf, gl1, u01, scale=True), layout)
            assert np.array_equal(gflat.cpu().numpy(), want_flat), ("pull", mode, rank, trial)
            gi, gt, gl = O.decode(want_flat, T)
            for c in cols:
                want = O.fused_subcopy(gimg, gi, gt, gl, stride, int(accu[c]), T, rows[c], off, Lm, head)
                assert np.array_equal(outs[c].cpu().numpy(), want), ("pull", mode, rank, trial, c)
        assert sampler.result()[1][0] == 0
        rp.disable_pull()
    if W > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print("SHARDED_GPU_OK", W)


if __name__ == "__main__":
    main()
