"""Head-sharded tensor-parallel mixers on two GPUs (NCCL all-reduce after out_proj) against the
reference's golden outputs.  Needs two devices; skipped otherwise."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from conftest import load_golden, rel_err
    from based_b200.generation import InferenceParams
    from based_b200.mixers import LinearAttention, TaylorExp
    from based_b200.sharding import shard_linear_attention_state_dict
    g = load_golden("linattn_mixer.npz")
    d_model, H, d, dv, B, L, steps = [int(x) for x in g["meta"]]
    full = {"proj_q.weight": g["wq"], "proj_k.weight": g["wk"], "proj_v.weight": g["wv"], "out_proj.weight": g["wo"]}
    m = LinearAttention(d_model=d_model, feature_map=TaylorExp(input_dim=d), feature_dim=d, num_heads=H,
                        head_dim=dv, layer_idx=0, process_group=dist.group.WORLD)
    m.load_state_dict(shard_linear_attention_state_dict(full, H, d, dv, rank, world))
    m = m.cuda()
    x = g["x"].cuda()
    errs = []
    with torch.inference_mode():
        ip = InferenceParams(max_seqlen=L + steps, max_batch_size=B)
        y = m(x[:, :L], inference_params=ip)
        errs.append(rel_err(y.cpu(), g["y_prefill"]))
        for s in range(steps):
            ip.seqlen_offset = L + s
            y = m(x[:, L + s:L + s + 1], inference_params=ip)
            errs.append(rel_err(y.cpu(), g["y_decode"][:, s:s + 1]))
        kv = ip.key_value_memory_dict[0][0]
        h0 = rank * (H // world)
        errs.append(rel_err(kv.cpu(), g["kv_state_final"][:, h0:h0 + H // world]))
    q.put((rank, max(errs), tuple(kv.shape)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_linear_attention_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 32500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert err < 1e-4, (rank, err)
        assert shape[1] == 1  # each rank holds one of the two heads of the state
