"""Tensor-parallel sharding arithmetic on CPU: two gloo ranks against the oracle.

Each rank asks the library for ITS schedule (``pi05_schedule_plan_tp``, host arithmetic only), reads off which rows of
wq / wg / wu and which columns of wo / wd that schedule streams, computes the partial sums of one expert layer's O and
down projections from exactly those slices (FP32, layer 0 of the full geometry, oracle inputs), and the ranks
all-reduce them the way the engines do on GPUs (a sum in rank order).  The result must equal the oracle's unsharded
layer (reference/pi05.py:254-265, 268-279) up to FP32 summation order, which shows that the shares the engine binds
are consistent: the heads a rank projects are the heads whose wo columns it owns, the MLP columns it activates are the
ones whose wd columns it owns, and the shares are disjoint and complete.
"""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import _lib, build
from pi05_megakernel_b200 import fixture as FX

QKV, OPROJ, GU, DOWN = range(4)


def shares(rank: int, size: int) -> dict:
    """Rows / columns a rank streams, from its schedule: q rows of wq, K columns of wo, rows of wg / wu, K columns of wd."""
    entries, _ = _lib.schedule_plan(148, 1, 128, rank, size)
    q_rows, o_cols, gu_rows, d_cols = set(), set(), set(), set()
    for _cta, gemm, _lag, _group, tile, k0, nk in entries:
        ks = range(k0 * 128, (k0 + nk) * 128)
        if gemm == QKV and tile < 16:
            q_rows.update(range(tile * 128, tile * 128 + 128))
        elif gemm == OPROJ:
            o_cols.update(ks)
        elif gemm == GU:
            gu_rows.update(range(tile * 64, tile * 64 + 64))
        elif gemm == DOWN:
            d_cols.update(ks)
    return {k: torch.tensor(sorted(v)) for k, v in dict(q=q_rows, o=o_cols, gu=gu_rows, d=d_cols).items()}


def _worker(rank: int, world: int, port: int, out) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    w = FX.make_weights(geo, 11)
    obs = FX.make_observation(geo, 11, "pad")
    f = lambda t: t.float()
    sh = shares(rank, world)
    positions, allowed = O.suffix_layout(obs["prefix_mask"], geo.horizon)
    cast = O._cast(True)
    an = torch.randn(geo.horizon, geo.hidden)                     # the normalised activations both GEMMs start from

    # ---- attention + O projection: this rank's heads only
    heads = sorted({int(r) // geo.head_dim for r in sh["q"]})
    assert sh["q"].numel() == len(heads) * geo.head_dim
    assert sorted(int(c) for c in sh["o"]) == [h * geo.head_dim + i for h in heads for i in range(geo.head_dim)]
    q = O.rope((an @ f(w["wq"][0])[sh["q"]].T).view(geo.horizon, len(heads), geo.head_dim), positions, cast)
    k = O.rope((an @ f(w["wk"][0]).T).view(geo.horizon, 1, geo.head_dim), positions, cast)
    v = (an @ f(w["wv"][0]).T).view(geo.horizon, 1, geo.head_dim)
    keys = torch.cat((f(obs["prefix_k"][0]), k))
    vals = torch.cat((f(obs["prefix_v"][0]), v))
    mixed = O.attention(q, keys, vals, allowed, cast).reshape(geo.horizon, -1)
    o_part = mixed @ f(w["wo"][0])[:, sh["o"]].T
    # ---- MLP: this rank's columns of the intermediate width
    assert torch.equal(sh["gu"], sh["d"])
    act = F.gelu(an @ f(w["wg"][0])[sh["gu"]].T, approximate="tanh") * (an @ f(w["wu"][0])[sh["gu"]].T)
    d_part = act @ f(w["wd"][0])[:, sh["d"]].T

    parts = [torch.zeros_like(o_part) for _ in range(world)]
    dist.all_gather(parts, o_part)
    o_sum = sum(parts[1:], parts[0])                             # rank order, as the engines add
    parts = [torch.zeros_like(d_part) for _ in range(world)]
    dist.all_gather(parts, d_part)
    d_sum = sum(parts[1:], parts[0])

    # ---- the unsharded layer
    values = {**{k_: f(v_) if v_.dtype == torch.bfloat16 else v_ for k_, v_ in w.items()},
              "prefix_k": f(obs["prefix_k"]), "prefix_v": f(obs["prefix_v"])}
    o_full = O.expert_attention(values, ogeo, 0, an, positions, allowed, True)
    d_full = (F.gelu(an @ f(w["wg"][0]).T, approximate="tanh") * (an @ f(w["wu"][0]).T)) @ f(w["wd"][0]).T
    rel = lambda a, b: float((a - b).norm() / b.norm())
    out.put((rank, rel(o_sum, o_full), rel(d_sum, d_full), len(heads), int(sh["gu"].numel())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_sum_to_the_unsharded_layer():
    build.build()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 31000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, o_err, d_err, nheads, ncols in results:
        assert nheads == 4 and ncols == 2048
        assert o_err < 1e-5 and d_err < 1e-5, (rank, o_err, d_err)
