"""Data parallelism around expert parallelism on CPU (gloo): expert parameters stay local, replicated ones are reduced;
model families run on the CPU backend."""
import torch
import torch.distributed as dist

from tests.mp_util import run_ranks


def _ddp_rank(rank, world):
    from ccfuser_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    from ccfuser_b200.parallel.ddp import expert_param_names, wrap_ddp
    torch.manual_seed(0)   # same replicated parameters everywhere
    c = GPTMoEConfig(vocab_size=128, n_layer=2, n_head=2, d_model=32, d_ffn=64, seq_len=16, num_experts=4, top_k=2,
                     ep_size=world, backend="cpu", max_tokens=32, dtype=torch.float32)
    model = GPTMoE(c)
    names = expert_param_names(model)
    ddp = wrap_ddp(model)
    ignored = set(getattr(model, "_ddp_params_and_buffers_to_ignore", []))
    g = torch.Generator().manual_seed(10 + rank)   # different data per rank
    ids = torch.randint(0, 128, (2, 16), generator=g)
    loss = ddp(ids, ids.roll(-1, 1))
    loss.backward()
    rep = model.h[0].attn.q_proj.weight.grad.clone()
    gate = model.h[1].mlp.gate.gate.weight.grad.clone()
    exp = model.h[1].mlp.experts.htoh4.weight.grad.clone()
    outs = []
    for t in (rep, gate, exp):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        outs.append(bool(torch.allclose(parts[0], parts[1])))
    return names, sorted(ignored), outs


def test_ddp_skips_expert_parameters():
    res = run_ranks(_ddp_rank, 2)
    names, ignored, (rep_equal, gate_equal, exp_equal) = res[0]
    assert names and all(".experts." in n for n in names)
    assert set(names) == set(ignored)
    assert rep_equal and gate_equal, "replicated parameters (attention, router) get the all-reduced gradient"
    assert not exp_equal, "expert gradients are local to the owning rank"


def test_all_model_families_step_on_cpu():
    from ccfuser_b200.examples import train
    import sys
    for model in ("gpt", "bert", "txl"):
        for variant in ("dense", "nccl"):
            argv = ["train", "--model", model, "--variant", variant, "--steps", "1", "--warmup", "0", "--layers", "2",
                    "--batch", "2", "--seq", "16", "--experts-per-gpu", "4", "--dtype", "bf16"]
            old = sys.argv
            sys.argv = argv
            try:
                train.main()
            finally:
                sys.argv = old


def test_lm_iterator_and_checkpoint_resume(tmp_path):
    import sys
    from ccfuser_b200.utils.data import LMOrderedIterator, synthetic_corpus
    from ccfuser_b200.examples import train
    data = synthetic_corpus(2000, 50, seed=1)
    it = LMOrderedIterator(data, batch_size=4, tgt_len=16)
    x0, y0 = it.get_batch(0)
    x1, _ = it.get_batch(1)
    assert x0.shape == (4, 16) and torch.equal(y0[:, :-1], x0[:, 1:]) and torch.equal(y0[:, -1], x1[:, 0])
    assert len(list(it)) == len(it) > 0
    # save after two steps, resume into a fresh process-local model: the first loss after resuming continues the run
    prefix = str(tmp_path / "ck")
    base = ["train", "--model", "gpt", "--variant", "nccl", "--warmup", "0", "--layers", "2", "--batch", "2", "--seq", "16",
            "--experts-per-gpu", "4", "--dtype", "bf16", "--lr", "0.05"]
    old = sys.argv
    try:
        sys.argv = base + ["--steps", "2", "--save", prefix]
        train.main()
        sys.argv = base + ["--steps", "1", "--resume", prefix]
        train.main()
        # a restarted job: same command line every time, periodic checkpoints, resume from whatever is there
        prefix2 = str(tmp_path / "job")
        restartable = base + ["--steps", "3", "--save", prefix2, "--save-every", "2", "--resume", prefix2]
        sys.argv = restartable
        train.main()                                   # first attempt: nothing to resume
        import json
        assert json.load(open(prefix2 + ".manifest.json"))["extra"]["step"] == 3
        sys.argv = restartable
        train.main()                                   # "restart": continues from step 3
        assert json.load(open(prefix2 + ".manifest.json"))["extra"]["step"] == 6
    finally:
        sys.argv = old
    import os
    assert os.path.exists(prefix + ".manifest.json") and os.path.exists(prefix + ".ep0of1.pt")


def _ep_dp_rank(rank, world):
    """4 ranks = 2 expert-parallel groups of 2 (ranks {0,1} and {2,3}) x 2 data-parallel replicas of every expert."""
    from ccfuser_b200 import MoEConfig, MoELayer
    from ccfuser_b200.parallel.ddp import allreduce_replicated_grads, reduce_expert_grads
    from ccfuser_b200.utils.dist import make_ep_dp_groups
    from tests.test_cpu_layer import _full_params, _inputs, load_shard
    ep_group, dp_group = make_ep_dp_groups(2)
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=None, activation="gelu",
                    dtype=torch.float32, ep_size=2, backend="cpu", max_tokens=64)
    layer = MoELayer(cfg, ep_group=ep_group)
    assert layer.ep_rank == rank % 2
    load_shard(layer, _full_params(cfg, 0), layer.ep_rank)
    x = _inputs(world, 64, 32)[rank]
    y = layer(x)
    (y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum().backward()
    allreduce_replicated_grads(layer, None, average=True)          # router: mean over all 4 ranks
    reduce_expert_grads(layer, dp_group, scale=1.0 / world)         # experts: sum over the 2 replicas, same convention
    return {n: p.grad.clone() for n, p in layer.named_parameters()}, dist.get_process_group_ranks(dp_group)


def test_expert_parallel_inside_data_parallel():
    from ccfuser_b200 import MoEConfig
    from ccfuser_b200.ops.reference import dense_moe_oracle
    from tests.test_cpu_layer import _full_params, _inputs
    world = 4
    res = run_ranks(_ep_dp_rank, world)
    cfg = MoEConfig(d_model=32, d_ffn=64, num_experts=4, top_k=2, capacity_factor=None, activation="gelu", dtype=torch.float32)
    full = {k: v.clone().requires_grad_(True) for k, v in _full_params(cfg, 0).items()}
    xs = _inputs(world, 64, 32)
    ys = dense_moe_oracle(xs, full, top_k=2, capacity=None, activation="gelu")
    (sum((y * torch.linspace(-1, 1, y.numel()).view_as(y)).sum() for y in ys) / world).backward()
    assert [res[r][1] for r in range(4)] == [[0, 2], [1, 3], [0, 2], [1, 3]]
    for r in range(world):
        grads = res[r][0]
        sl = slice((r % 2) * 2, (r % 2) * 2 + 2)
        assert torch.allclose(grads["gate.gate.weight"], full["gate.weight"].grad, atol=1e-6, rtol=1e-4)
        for name in ("htoh4", "h4toh"):
            assert torch.allclose(grads[f"experts.{name}.weight"], full[name + ".weight"].grad[sl], atol=1e-6, rtol=1e-4)
            assert torch.allclose(grads[f"experts.{name}.bias"], full[name + ".bias"].grad[sl], atol=1e-6, rtol=1e-4)


def test_example_trainer_with_two_expert_parallel_groups():
    """4 CPU ranks as 2 expert-parallel groups x 2 replicas through the example trainer's command line."""
    import json
    import os
    import subprocess
    import sys
    from tests.mp_util import _free_port
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "ccfuser_b200.examples.train", "--model", "gpt", "--variant", "nccl", "--ep-size", "2",
           "--steps", "2", "--warmup", "0", "--layers", "2", "--batch", "2", "--seq", "16", "--experts-per-gpu", "2"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    out = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    rec = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")][-1]
    assert rec["n_gpus"] == 4 and rec["final_loss"] == rec["final_loss"]      # finite


def test_vocab_and_corpus(tmp_path):
    from ccfuser_b200.utils.data import Corpus
    train = tmp_path / "train.txt"
    train.write_text("the cat sat on the mat\nthe dog sat\n\nA cat\n")
    corpus = Corpus(str(train), valid=["the bird sat"], lower=True, min_freq=1)
    v = corpus.vocab
    assert v.idx2sym[:2] == ["<unk>", "<eos>"] and v.idx2sym[2] == "the"          # most frequent word first
    assert len(v) == 2 + len({"the", "cat", "sat", "on", "mat", "dog", "a"})
    ids = corpus.data["train"]
    assert v.decode(ids[:7]) == "the cat sat on the mat <eos>" and int((ids == v.sym2idx["<eos>"]).sum()) == 3
    assert v.decode(corpus.data["valid"]) == "the <unk> sat <eos>"
    it = corpus.iterator("train", batch_size=2, tgt_len=3)
    x, y = next(iter(it))
    assert x.shape == (2, 3) and torch.equal(x[:, 1:], y[:, :-1])
    small = Corpus(["a a a b b c"], max_size=4, add_eos=False)
    assert small.vocab.idx2sym == ["<unk>", "a", "b", "c"]


def test_txl_example_trains_from_a_text_file(tmp_path, capsys):
    import json
    import random
    import sys
    from ccfuser_b200.examples import train
    rnd = random.Random(0)
    words = ["w%d" % i for i in range(40)]
    (tmp_path / "train.txt").write_text("\n".join(" ".join(rnd.choice(words) for _ in range(12)) for _ in range(200)))
    (tmp_path / "valid.txt").write_text("\n".join(" ".join(rnd.choice(words) for _ in range(12)) for _ in range(40)))
    old = sys.argv
    sys.argv = ["train", "--model", "txl", "--variant", "nccl", "--steps", "4", "--warmup", "0", "--layers", "2", "--batch", "4",
                "--seq", "16", "--experts-per-gpu", "4", "--lr", "0.05", "--data", str(tmp_path / "train.txt"),
                "--valid", str(tmp_path / "valid.txt")]
    try:
        train.main()
    finally:
        sys.argv = old
    recs = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert recs[0]["final_loss"] == recs[0]["final_loss"]
    assert recs[1]["vocab"] == 42 and recs[1]["valid_loss"] > 0


def test_checkpoint_carries_optimizer_state(tmp_path):
    from ccfuser_b200 import MoEConfig, MoELayer, load_ep_checkpoint, save_ep_checkpoint
    torch.manual_seed(0)
    cfg = MoEConfig(d_model=16, d_ffn=32, num_experts=4, dtype=torch.float32, backend="cpu")
    layer = MoELayer(cfg)
    opt = torch.optim.AdamW(layer.parameters(), lr=1e-2)
    x = torch.randn(20, 16)
    for _ in range(3):
        opt.zero_grad()
        layer(x).square().sum().backward()
        opt.step()
    prefix = str(tmp_path / "ck")
    save_ep_checkpoint(layer, prefix, 0, 1, optimizer=opt, extra={"step": 3})
    layer2 = MoELayer(cfg)
    opt2 = torch.optim.AdamW(layer2.parameters(), lr=1e-2)
    manifest = load_ep_checkpoint(layer2, prefix, 0, 1, optimizer=opt2)
    assert manifest["optimizer_restored"] and manifest["extra"]["step"] == 3
    for a, b in zip(layer.parameters(), layer2.parameters()):
        assert torch.equal(a, b)
        assert torch.equal(opt.state[a]["exp_avg_sq"], opt2.state[b]["exp_avg_sq"])
    # the next step is identical on both
    for l, o in ((layer, opt), (layer2, opt2)):
        o.zero_grad()
        l(x).square().sum().backward()
        o.step()
    assert all(torch.equal(a, b) for a, b in zip(layer.parameters(), layer2.parameters()))
    # another expert-parallel degree: parameters re-sharded, optimizer starts fresh
    cfg2 = cfg.replace(num_experts=4)
    assert load_ep_checkpoint(MoELayer(cfg2), prefix, 0, 1, optimizer=None)["ep_size"] == 1
