"""ops/optim.py on the host: the torch fallback of FusedSGD and the launch table it fills for the multi-tensor kernel."""
import ctypes as C

import torch

from ccfuser_b200 import native as N
from ccfuser_b200.ops.optim import FusedSGD


def test_cpu_parameters_take_the_torch_path_and_match_torch_sgd():
    torch.manual_seed(0)
    ours = [torch.nn.Parameter(torch.randn(7, 5)), torch.nn.Parameter(torch.randn(3))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in ours]
    for a, b in zip(ours, ref):
        g = torch.randn_like(a)
        a.grad, b.grad = g.clone(), g.clone()
    FusedSGD(ours, lr=0.1, weight_decay=0.01).step()
    torch.optim.SGD(ref, lr=0.1, weight_decay=0.01).step()
    for a, b in zip(ours, ref):
        assert torch.allclose(a, b, atol=1e-6)


class _FakeTensor:
    def __init__(self, ptr, n):
        self._ptr, self._n = ptr, n

    def data_ptr(self):
        return self._ptr

    def numel(self):
        return self._n


class _FakeLib:
    def __init__(self):
        self.tables = []

    def ccf_sgd_multi(self, table_ref, stream):
        t = table_ref._obj
        self.tables.append(N.SgdMulti.from_buffer_copy(bytes(t)))
        return 0


def test_launch_table_gives_every_tensor_its_blocks():
    opt = FusedSGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1)
    lib = _FakeLib()
    sizes = [1, 8191, 8192, 8193, 10 ** 9]
    batch = [(_FakeTensor(0x1000 * (i + 1), n), _FakeTensor(0x2000 * (i + 1), n)) for i, n in enumerate(sizes)]
    opt._launch(lib, batch, 0.25, 0.5, 1, None)
    t = lib.tables[0]
    assert t.count == len(sizes) and abs(t.lr - 0.25) < 1e-7 and abs(t.wd - 0.5) < 1e-7 and t.fp16 == 1
    blocks = [t.first_block[i + 1] - t.first_block[i] for i in range(len(sizes))]
    assert t.first_block[0] == 0
    assert blocks == [1, 1, 1, 2, 148 * 16]            # 8192 elements per block, capped for very large tensors
    assert [t.n[i] for i in range(len(sizes))] == sizes
    assert [t.p[i] for i in range(len(sizes))] == [0x1000 * (i + 1) for i in range(len(sizes))]
    assert C.sizeof(N.SgdMulti) == 48 * 24 + 49 * 4 + 16 + 4      # the layout the library checks at load time


def test_closure_runs_with_gradients_enabled():
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    opt = FusedSGD([p], lr=0.5)

    def closure():
        opt.zero_grad()
        loss = (p * p).sum()
        loss.backward()
        return loss

    loss = opt.step(closure)
    assert float(loss) == 5.0 and torch.allclose(p.detach(), torch.tensor([0.0, 0.0]))
