"""The KV-range split with the merge over peer memory (b200kv_peer_merge). On one GPU the exchange
degenerates to a single rank; with two or more GPUs the test starts one process per GPU, each attends over
its block range of one sequence, pushes its partial into every rank's exchange buffer and merges, several
layers in a row (the epoch on the device advances), eagerly and from a replayed CUDA graph. Every rank's
result is held against the float64 reference of the whole sequence."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import b200kv
import kvo
import scenarios
from gpu_util import from_dev_bf16, to_dev_bf16, to_dev_i32

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "ascend-moe-engine_b200")); sys.path.insert(0, os.path.join(ROOT, "tests"))
import numpy as np, torch, torch.distributed as dist
import b200kv, kvo, scenarios
from b200kv import dist as kvdist
from gpu_util import from_dev_bf16, to_dev_bf16, to_dev_i32

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group(backend="nccl", device_id=torch.device("cuda", rank))
bs, n, layers, heads = 64, 64 * 37 + 11, 3, 64
blocks = scenarios.blocks_for(n, bs)
table = kvo.permutation(blocks)[None, :].astype(np.int32)
begin, length = kvdist.split_kv_range(n, bs, world, rank)
q_np = kvo.make_q(1)
pools = [kvo.make_pool(blocks * bs, seed=kvo.BASE_SEED + l) for l in range(layers)]
refs = [scenarios.ref_attention_f64(q_np, pools[l], table, np.array([n], dtype=np.int32), bs, 1.0 / 24.0) for l in range(layers)]
q = to_dev_bf16(q_np)
d_pools = [to_dev_bf16(p) for p in pools]      # every rank holds the whole pool here; it reads only its range
d_table, d_len, d_begin = to_dev_i32(table), to_dev_i32([length]), to_dev_i32([begin])
ws = torch.empty(b200kv.decode_workspace_bytes(1), dtype=torch.uint8, device="cuda")
po = torch.zeros((1, heads, 512), dtype=torch.float32, device="cuda")
pm = torch.zeros((1, heads), dtype=torch.float32, device="cuda")
pl = torch.zeros((1, heads), dtype=torch.float32, device="cuda")
outs = [torch.zeros((heads, 512), dtype=torch.bfloat16, device="cuda") for _ in range(layers)]
lses = [torch.zeros((heads,), dtype=torch.float32, device="cuda") for _ in range(layers)]
status = b200kv.new_status()
exchange = kvdist.PeerExchange(heads)
FUSED = os.environ.get("PEER_FUSED") == "1"   # b200kv_mla_decode_peer instead of decode + b200kv_peer_merge

def step():
    for l in range(layers):
        if FUSED:
            exchange.decode_merge(q, b200kv.pool_view(d_pools[l]), d_table, d_len, bs, 1.0 / 24.0, outs[l].view(1, heads, 512),
                                  lse=lses[l], kv_begin=d_begin, workspace=ws, status=status,
                                  max_ctas=(0, 5, 1)[l % 3])
            continue
        b200kv.mla_decode(q, b200kv.pool_view(d_pools[l]), d_table, d_len, bs, 1.0 / 24.0, kv_begin=d_begin,
                          partial=(po, pm, pl), workspace=ws, status=status)
        exchange.merge(po.view(heads, 512), pm.view(heads), pl.view(heads), outs[l], lses[l], status=status)

def check(what):
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0, status.cpu().tolist()
    for l in range(layers):
        scenarios.check_attention(from_dev_bf16(outs[l])[None], lses[l].cpu().numpy()[None], refs[l][0], refs[l][1],
                                  what=f"{what}, rank {rank}, layer {l}")
        outs[l].zero_()

step(); check("eager")
step(); check("eager again")
side = torch.cuda.Stream()
side.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(side):
    step()
torch.cuda.current_stream().wait_stream(side)
check("side stream")
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph):
    step()
check("capture")   # capture does not run the kernels: outputs are still zero, so this must be skipped below
'''


def _run_workers(world, tmp_path, fused=False):
    script = tmp_path / "peer_worker.py"
    body = WORKER.replace('check("capture")   # capture does not run the kernels: outputs are still zero, so this must be skipped below',
                          'torch.cuda.synchronize()\nfor _ in range(3):\n    graph.replay()\n    check("graph replay")\ndist.barrier()\nexchange.close()\ndist.destroy_process_group()\nprint("PEER_OK", rank)')
    script.write_text(f"ROOT = {ROOT!r}\n" + body)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29534" if fused else "29533", WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0", PEER_FUSED="1" if fused else "0")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outputs.append(out)
    for r, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0 and f"PEER_OK {r}" in out, f"rank {r} failed:\n{out[-3000:]}"


def test_peer_merge_single_rank_matches_lse_merge():
    """world = 1: the push goes to the rank's own inbox; result equals the plain merge of the same partial."""
    from b200kv import dist as kvdist

    heads = 64
    po = torch.randn((heads, 512), dtype=torch.float32, device="cuda")
    pm = torch.randn((heads,), dtype=torch.float32, device="cuda")
    pl = torch.rand((heads,), dtype=torch.float32, device="cuda") + 0.5
    exchange = kvdist.PeerExchange(heads)
    out = torch.zeros((heads, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((heads,), dtype=torch.float32, device="cuda")
    ref = torch.zeros_like(out)
    ref_lse = torch.zeros_like(lse)
    st = b200kv.new_status()
    for _ in range(3):  # three epochs through both inbox halves
        out.zero_()
        exchange.merge(po, pm, pl, out, lse, status=st)
        b200kv.lse_merge(po.view(1, heads, 512), pm.view(1, heads), pl.view(1, heads), ref, ref_lse)
        torch.cuda.synchronize()
        assert st.cpu().tolist()[0] == 0
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)) and torch.allclose(lse, ref_lse, atol=1e-6)
    exchange.close()


@pytest.mark.parametrize("fused", [False, True], ids=["decode_then_merge", "decode_peer"])
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_merge_two_ranks(tmp_path, fused):
    _run_workers(2, tmp_path, fused)


@pytest.mark.parametrize("fused", [False, True], ids=["decode_then_merge", "decode_peer"])
@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_peer_merge_four_ranks(tmp_path, fused):
    _run_workers(4, tmp_path, fused)


@pytest.mark.parametrize("max_ctas", [0, 7, 1])
def test_decode_peer_single_rank_equals_decode(max_ctas):
    """b200kv_mla_decode_peer with one rank: the merge kernel pushes into its own inbox and merges one shard, so
    the result must equal b200kv_mla_decode's on the same inputs (bit for bit where both merge the same parts),
    through several epochs and for a shard selected by kv_begin; sequences whose shard is empty give zeros."""
    from b200kv import dist as kvdist

    bs = 64
    kv_len = np.array([64 * 30 + 5, 0, 700], dtype=np.int32)
    kv_begin = np.array([64 * 3, 0, 0], dtype=np.int32)
    B = len(kv_len)
    blocks = int(sum(scenarios.blocks_for(int(b + n), bs) for b, n in zip(kv_begin, kv_len))) + 4
    table = scenarios.fragmented_tables(kv_begin + kv_len, bs, blocks)
    pool_np = kvo.make_pool(blocks * bs)
    q_np = kvo.make_q(B, scale=2.0 / 24.0)
    pool, q = to_dev_bf16(pool_np), to_dev_bf16(q_np)
    tbl, lens, begins = to_dev_i32(table), to_dev_i32(kv_len), to_dev_i32(kv_begin)
    ws = torch.empty(b200kv.decode_workspace_bytes(B, 64, max_ctas), dtype=torch.uint8, device="cuda")
    exchange = kvdist.PeerExchange(B * 64)
    status = b200kv.new_status()
    ref_out, ref_lse = scenarios.ref_attention_f64(q_np, pool_np, table, kv_len, bs, 1.0 / 24.0, kv_begin=kv_begin)
    for epoch in range(3):
        out = torch.full((B, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((B, 64), float("nan"), dtype=torch.float32, device="cuda")
        exchange.decode_merge(q, b200kv.pool_view(pool), tbl, lens, bs, 1.0 / 24.0, out, lse=lse.view(-1), kv_begin=begins,
                              workspace=ws, max_ctas=max_ctas, status=status)
        torch.cuda.synchronize()
        assert status.cpu().tolist()[0] == 0, status.cpu().tolist()
        scenarios.check_attention(from_dev_bf16(out), lse.cpu().numpy(), ref_out, ref_lse,
                                  what=f"decode_peer, one rank, epoch {epoch}, max_ctas {max_ctas}")
        assert (from_dev_bf16(out)[1] == 0).all()
    exchange.close()
    # refused where it cannot run
    big_q = to_dev_bf16(kvo.make_q(16))
    with pytest.raises(b200kv.B200KVError):
        kvdist.PeerExchange(16 * 64).decode_merge(big_q, b200kv.pool_view(pool), to_dev_i32(np.zeros((16, 4))),
                                                  to_dev_i32(np.zeros(16)), bs, 1.0 / 24.0,
                                                  torch.zeros((16, 64, 512), dtype=torch.bfloat16, device="cuda"),
                                                  workspace=ws)


def test_peer_merge_wait_runs_out_when_a_peer_never_arrives():
    """A rank whose peer never pushes: the wait for the peer's words is bounded (about a second), the kernel
    returns with B200KV_DEV_TIMEOUT in the status word, and the GPU context stays usable. The missing peer is
    a second exchange buffer on the same GPU that nothing ever writes to; nothing faults or hangs."""
    import ctypes
    import time
    from ctypes import c_void_p

    from b200kv import dist as kvdist  # declares the argument types

    lib = b200kv.lib
    rows, world = 64, 2
    nbytes = lib.b200kv_peer_exchange_bytes(world, rows)
    assert nbytes > 2 * world * rows * 514 * 8
    bufs, handle = [], (ctypes.c_ubyte * 64)()
    for _ in range(world):
        ptr = c_void_p()
        b200kv.check(lib.b200kv_peer_buffer_alloc(nbytes, ctypes.byref(ptr), handle))
        bufs.append(ptr)
    table = (c_void_p * world)(bufs[0].value, bufs[1].value)
    po = torch.randn((rows, 512), dtype=torch.float32, device="cuda")
    pm = torch.zeros((rows,), dtype=torch.float32, device="cuda")
    pl = torch.ones((rows,), dtype=torch.float32, device="cuda")
    out = torch.full((rows, 512), 5.0, dtype=torch.bfloat16, device="cuda")
    st = b200kv.new_status()
    torch.cuda.synchronize()
    t0 = time.time()
    b200kv.check(lib.b200kv_peer_merge(table, world, 0, rows, po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                                       None, None, st.data_ptr()))
    torch.cuda.synchronize()
    waited = time.time() - t0
    status = st.cpu().tolist()
    assert status[0] == b200kv.DEV_TIMEOUT and status[1] == 50 and status[2] == 1, status   # site 50, source rank 1
    assert 0.5 < waited < 10.0, waited
    assert bool((out == 5.0).all())                       # nothing was merged
    # the context is alive and the same buffers work once the "peer" is the rank itself
    single = (c_void_p * 1)(bufs[1].value)
    st2 = b200kv.new_status()
    b200kv.check(lib.b200kv_peer_merge(single, 1, 0, rows, po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                                       None, None, st2.data_ptr()))
    torch.cuda.synchronize()
    assert st2.cpu().tolist()[0] == 0
    assert torch.allclose(out.float(), po, atol=0.02, rtol=0.01)
    for ptr in bufs:
        b200kv.check(lib.b200kv_peer_buffer_free(ptr))
