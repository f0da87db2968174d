"""Host-side logic of the multi-GPU benchmark, on CPU: two gloo ranks build their shards of the batched workload (by frame)
and of the divergent launch (by plane); the shards are disjoint, cover the job, and reduce to the timing the benchmark
reports (max over ranks)."""
import os
import socket
import subprocess
import sys
import textwrap

from conftest import ROOT

WORKER = textwrap.dedent('''
    import os, sys, json
    sys.path.insert(0, sys.argv[1])
    import torch, torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    out = {}
    for scaling in ("weak", "strong"):
        wl, frames = bench.shard_workload(rank, world, scaling, n_frames=8, frame_w=96, frame_h=64)
        seeds = [int(s[:8].sum()) + int(s[-8:].sum()) * 7 for s in wl.sources]          # fingerprints of the frames
        rects = [p.crop for p in wl.planes]
        gathered = [None] * world
        dist.all_gather_object(gathered, {"frames": frames, "n_src": len(wl.sources), "n_planes": len(wl.planes),
                                          "px": wl.out_pixels, "seeds": seeds, "rects": rects})
        out[scaling] = gathered
    from fusedkernellibrary_b200 import workloads as W
    whole = W.divergent_planes(n_per_seq=4, w=64, h=32)
    mine = W.shard_by_plane(whole, rank, world)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"global_planes": mine.extra["global_planes"], "chains": [p.chain for p in mine.planes],
                                      "dst": [(p.dst, p.dst_offset) for p in mine.planes], "n_src": len(mine.sources),
                                      "out_sizes": mine.out_sizes,
                                      "frames": [int(s[:16].sum()) * 31 + int(s[-16:].sum()) for s in mine.sources]})
    out["config5"] = gathered
    out["config5_whole"] = {"dst": [(p.dst, p.dst_offset) for p in whole.planes], "out_sizes": whole.out_sizes, "n_planes": len(whole.planes)}
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out["max_time"] = float(t.item())
    if rank == 0:
        print("RESULT " + json.dumps(out))
    dist.destroy_process_group()
''')


def test_two_rank_sharding_with_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), ROOT]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][0]
    res = json.loads(line[len("RESULT "):])
    assert res["max_time"] == 2.0  # the slowest rank's time is the one reported
    weak, strong = res["weak"], res["strong"]
    # weak: every rank runs the whole workload on its own frames
    assert [g["frames"] for g in weak] == [8, 8] and [g["n_planes"] for g in weak] == [8 * 32] * 2
    assert set(weak[0]["seeds"]).isdisjoint(weak[1]["seeds"])
    # strong: the frames of one job are split by frame; shards are disjoint and cover it
    assert [g["frames"] for g in strong] == [4, 4] and sum(g["n_planes"] for g in strong) == 8 * 32
    assert set(strong[0]["seeds"]).isdisjoint(strong[1]["seeds"])
    assert strong[0]["rects"] != strong[1]["rects"]
    assert sum(g["px"] for g in strong) == weak[0]["px"]
    # the divergent launch split by plane: the ranks' planes are disjoint and cover the launch, every rank gets as many
    # planes of the first chain as of the second, a plane keeps its place in output tensors of the global shape (the
    # reference hands every sequence the global plane index), and a rank holds only the frames its planes read
    c5, whole5 = res["config5"], res["config5_whole"]
    planes = sorted(z for g in c5 for z in g["global_planes"])
    assert planes == list(range(whole5["n_planes"]))
    for g in c5:
        assert g["chains"].count(0) == g["chains"].count(1) == 2
        assert g["out_sizes"] == whole5["out_sizes"]
        assert [tuple(d) for d in g["dst"]] == [tuple(whole5["dst"][z]) for z in g["global_planes"]]
        assert g["n_src"] == len(g["global_planes"])
    assert set(c5[0]["frames"]).isdisjoint(c5[1]["frames"])
