"""Flag protocol (host emulation), host-side failure detection, checkpoint re-sharding. CPU only; no GPU is
faulted or hung by any of these tests."""
import os
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist

from ccfuser_b200 import MoECommTimeout
from ccfuser_b200.parallel.flag_protocol import EmulatedRank, run_call, TILE
from ccfuser_b200.ops.routing import route_local, global_plan
from tests.mp_util import run_ranks


def _make_plans(world, tokens, e_loc, k, d, seed):
    rng = np.random.RandomState(seed)
    e_tot = world * e_loc
    idxs = [torch.from_numpy(np.stack([rng.permutation(e_tot)[:k] for _ in range(tokens)])) for _ in range(world)]
    locs = [route_local(i, e_tot, tokens * k) for i in idxs]
    table = torch.stack([l.count for l in locs])
    gp = global_plan(table, e_loc, TILE)
    plans = []
    for r in range(world):
        loc = locs[r]
        row = gp.expert_base[loc.expert] + gp.src_offset[r][loc.expert] + loc.pos
        tiles = []
        for e in range(r * e_loc, (r + 1) * e_loc):
            n, base = int(gp.expert_rows[e]), int(gp.expert_base[e])
            for i in range((n + TILE - 1) // TILE):
                tiles.append((base // TILE + i, min(TILE, n - i * TILE)))
        plans.append({"x": rng.randn(tokens, d).astype(np.float32), "slot_owner": (loc.expert // e_loc).numpy(),
                      "slot_row": row.numpy(), "top_k": k, "tiles": tiles})
    return plans, int(gp.rank_rows.max())


def test_protocol_out_of_order_arrival_and_two_calls():
    world, tokens, e_loc, k, d = 4, 96, 2, 2, 8
    plans, max_rows = _make_plans(world, tokens, e_loc, k, d, 0)
    ranks = [EmulatedRank(r, world, max_rows + TILE, tokens * k, d) for r in range(world)]
    fn = lambda owner, row, x: 2.0 * x + owner
    for call in range(2):  # the second call reuses every buffer and counter
        outs = run_call(ranks, plans, fn, timeout_s=5.0, shuffle_seed=call)
        for r in range(world):
            owners = plans[r]["slot_owner"].reshape(tokens, k)
            ref = sum(2.0 * plans[r]["x"] + owners[:, j:j + 1] for j in range(k))
            assert np.allclose(outs[r], ref)
        assert all((rk.tile_flags == 0).all() for rk in ranks)


def test_protocol_missing_sender_times_out():
    world, tokens, e_loc, k, d = 2, 64, 2, 2, 4
    plans, max_rows = _make_plans(world, tokens, e_loc, k, d, 1)
    ranks = [EmulatedRank(r, world, max_rows + TILE, tokens * k, d) for r in range(world)]
    t0 = time.monotonic()
    with pytest.raises(MoECommTimeout):
        run_call(ranks, plans, lambda o, row, x: x, timeout_s=0.3, drop_sender=1)
    assert time.monotonic() - t0 < 10


def test_early_token_of_next_call_does_not_satisfy_current_wait():
    me = EmulatedRank(0, 2, TILE, 8, 2)
    # owner 1 is one call ahead: it already delivered call 1's rows + token AND call 2's token, owner 0 nothing yet
    me.done[1] = (3 * 2 + 1) + 1
    with pytest.raises(MoECommTimeout) as ei:
        me.wait_combine([2, 3], units=2, timeout_s=0.2)
    assert ei.value.peer == 0
    me.done[0] = 2 * 2 + 1
    me.wait_combine([2, 3], units=2, timeout_s=0.2)
    assert list(me.done_cum) == [5, 7]
    # the early token is still there for the next call
    me.done[0] += 1
    me.wait_combine([0, 0], units=2, timeout_s=0.2)


def _rank_that_leaves(rank, world, store_path):
    from ccfuser_b200.utils.watchdog import Heartbeat
    store = dist.FileStore(store_path, world)
    hb = Heartbeat(store, rank, world)
    hb.beat(0)
    hb.check(0, timeout_s=20)
    if rank == 1:
        return "left"            # leaves between steps, nothing in flight
    hb.beat(1)
    try:
        hb.check(1, timeout_s=1.0)
    except MoECommTimeout as e:
        return f"timeout peer={e.peer}"
    return "no error"


def test_heartbeat_reports_rank_that_left(tmp_path):
    res = run_ranks(_rank_that_leaves, 2, str(tmp_path / "store"))
    assert res[1] == "left" and res[0] == "timeout peer=1"


def _collective_with_missing_rank(rank, world):
    from ccfuser_b200.utils.watchdog import run_with_timeout
    x = torch.ones(4)
    if rank == 1:
        time.sleep(3.0)          # never joins the collective in time
        return "late"
    try:
        run_with_timeout(lambda: dist.all_reduce(x), 1.0, "all_reduce")
    except MoECommTimeout as e:
        return "timeout " + str(e.where)
    return "no error"


def test_bounded_collective_times_out_cleanly():
    res = run_ranks(_collective_with_missing_rank, 2)
    assert res[0] == "timeout all_reduce"


def test_checkpoint_reshard_round_trip(tmp_path):
    from ccfuser_b200 import MoEConfig, MoELayer
    from ccfuser_b200.utils.checkpoint import ep_state_dict, reshard_expert_state, save_ep_checkpoint, load_ep_checkpoint
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=16, d_ffn=32, num_experts=8, top_k=2, dtype=torch.float32, ep_size=1, backend="cpu")
    full = MoELayer(cfg)
    parts = ep_state_dict(full)
    assert set(parts["experts"]) == {"experts.htoh4.weight", "experts.htoh4.bias", "experts.h4toh.weight", "experts.h4toh.bias"}
    assert set(parts["replicated"]) == {"gate.gate.weight", "gate.gate.bias"}
    s4 = reshard_expert_state([parts["experts"]], 4)
    assert s4[2]["experts.htoh4.weight"].shape == (2, 32, 16)
    s2 = reshard_expert_state(s4, 2)
    s1 = reshard_expert_state(s2, 1)
    for k, v in parts["experts"].items():
        assert torch.equal(s1[0][k], v)
        assert torch.equal(s2[1][k], v[4:])
    # files: save at EP=1, load into an identical model; then emulate a 4-way save and load back at EP=1
    prefix = str(tmp_path / "ckpt")
    save_ep_checkpoint(full, prefix, 0, 1)
    other = MoELayer(cfg)
    load_ep_checkpoint(other, prefix, 0, 1)
    x = torch.randn(10, 16)
    assert torch.equal(full(x), other(x))
    import json
    for r in range(4):
        torch.save(s4[r], f"{prefix}4.ep{r}of4.pt")
    torch.save(parts["replicated"], f"{prefix}4.replicated.pt")
    json.dump({"ep_size": 4, "experts_per_rank": {}, "expert_keys": [], "extra": {}}, open(f"{prefix}4.manifest.json", "w"))
    third = MoELayer(cfg)
    load_ep_checkpoint(third, prefix + "4", 0, 1)
    assert torch.equal(full(x), third(x))


def test_protocol_model_all_interleavings_are_safe():
    """Exhaustive exploration of the abstract protocol: forward passes exchange counts, backward passes do not."""
    from ccfuser_b200.parallel.protocol_model import check
    assert check(world=2, calls=4, chunks=2) > 100
    assert check(world=3, calls=4, chunks=1) > 1000
    assert check(world=4, calls=2, chunks=1) > 10000
    # uneven traffic, including a pair that exchanges nothing
    assert check(world=3, calls=2, chunks=1, rows=[[2, 0, 1], [0, 3, 1], [1, 1, 0]]) > 500
    # every call planned (inference: forward passes only) and no call planned after the first
    assert check(world=2, calls=3, chunks=1, plan_every=1) > 50
    assert check(world=2, calls=3, chunks=1, plan_every=100) > 50


def test_protocol_model_split_token_refinement_is_safe():
    """Token in its own counter, checked per owner right before the next push: lets an owner keep using its buffers
    after it has returned the rows. Safe in every interleaving, and strictly more concurrent than the current protocol."""
    from ccfuser_b200.parallel.protocol_model import check
    assert check(world=2, calls=4, chunks=1, variant="split_token") > check(world=2, calls=4, chunks=1)
    assert check(world=3, calls=4, chunks=1, variant="split_token") > 5000
    assert check(world=2, calls=4, chunks=2, variant="split_token", plan_every=100) > 500


def test_protocol_model_finds_the_hazards_of_broken_variants():
    import pytest
    from ccfuser_b200.parallel.protocol_model import ProtocolViolation, check
    for variant, what in (("token_before_store", "still uses the buffers"), ("no_token", "still uses the buffers"),
                          ("absolute_targets", "before owner"), ("reset_after_finish", "arrival is lost")):
        with pytest.raises(ProtocolViolation, match=what):
            check(world=2, calls=2, chunks=1, variant=variant)
