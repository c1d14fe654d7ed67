import numpy as np
import torch

from rocwmma_b200 import datagen as G


def test_generator_is_counter_based():
    a = G.raw_np(3, 1000)
    b = G.raw_np(3, 10, start=500)
    assert np.array_equal(a[500:510], b)
    assert len(np.unique(a)) == 1000


def test_numpy_and_torch_streams_agree():
    n = 4096
    for kind, ref in (("uniform", G.uniform_np(5, (n,), np.float32)), ("int8", G.int8_np(5, (n,))),
                      ("int4", G.int4_np(5, (n,)))):
        dt = torch.float32 if kind == "uniform" else torch.int8
        t = G.fill_torch(torch.empty(n, dtype=dt), 5, kind, chunk=1000)
        assert np.array_equal(t.numpy(), ref), kind
    t = G.fill_torch(torch.empty(n, dtype=torch.float16), 7, "normal", sigma=0.25, chunk=999)
    ref = G.normal_np(7, (n,), 0.25, np.float16)
    # same integer stream; libm differences may move a value by one fp16 ulp at most
    assert np.abs(t.numpy().astype(np.float32) - ref.astype(np.float32)).max() <= 2.0 ** -11


def test_distributions():
    u = G.uniform_np(1, (1 << 16,), np.float32)
    assert -1.0 <= u.min() and u.max() < 1.0 and abs(u.mean()) < 0.02
    g = G.normal_np(4, (1 << 16,), 0.25, np.float32)
    assert abs(g.std() - 0.25) < 0.01
    i = G.int8_np(2, (1 << 16,))
    assert i.min() == -128 and i.max() == 127
