"""The persistent kernel that runs a chain of decode-shaped products (csrc/decode_chain.cu), alone: the
four products between one layer's attention and the next (output projection with the residual add and the
norm's weight, gate/up with SwiGLU, down with the residual add, the next projection behind its norm) against
the same arithmetic in float64 with the same roundings, at the 1B widths and at sizes that divide by
nothing; the same through the kernels that run one by one; rows that do not depend on their batch."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def chains_on():
    """Chains are off by default (they are slower than single launches so far); these tests switch them on."""
    from picolm_b200.ops import chain
    old = chain.ENABLED
    chain.ENABLED = True
    yield
    chain.ENABLED = old


def _case(T, K0, d, F, N2, seed):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g)                                        # noqa: E731
    return {
        "a": (rnd(T, K0) / K0 ** 0.25).to(torch.bfloat16), "w1": (rnd(d, K0) / K0 ** 0.25).to(torch.bfloat16),
        "x": rnd(T, d) * torch.linspace(0.3, 4.0, T)[:, None], "nw1": (1.0 + 0.3 * rnd(d)).to(torch.bfloat16),
        "gate": (rnd(F, d) / d ** 0.5).to(torch.bfloat16), "up": (rnd(F, d) / d ** 0.5).to(torch.bfloat16),
        "down": (rnd(d, F) / F ** 0.5).to(torch.bfloat16), "nw2": (1.0 + 0.3 * rnd(d)).to(torch.bfloat16),
        "wq": (rnd(N2, d) / d ** 0.5).to(torch.bfloat16),
    }


def _reference(c, eps):
    b16 = lambda t: t.to(torch.bfloat16).double()                                        # noqa: E731
    x1 = c["x"].double() + c["a"].double() @ c["w1"].double().t()
    x1 = x1.float().double()                                                             # the stream is fp32
    r1 = 1.0 / torch.sqrt((x1 * x1).mean(dim=1, keepdim=True) + eps)
    xw1 = b16(x1 * c["nw1"].double())
    gate, up = b16(xw1 @ c["gate"].double().t() * r1), b16(xw1 @ c["up"].double().t() * r1)
    h = b16(gate / (1 + torch.exp(-gate)) * up)
    x2 = (x1 + h @ c["down"].double().t()).float().double()
    r2 = 1.0 / torch.sqrt((x2 * x2).mean(dim=1, keepdim=True) + eps)
    q = b16(b16(x2 * c["nw2"].double()) @ c["wq"].double().t() * r2)
    return x2, q, h @ c["down"].double().t()


def _run(c, eps, last="scaled"):
    from picolm_b200 import ops
    d = {k: v.to(DEV) for k, v in c.items()}
    x = d["x"].clone()
    w_gu = ops.interleave_gate_up(d["gate"], d["up"])
    p = ops.linear(d["a"], d["w1"], torch.float32, defer=True)
    s1 = ops.linear_residual_norm(p, x, d["nw1"], eps)
    h = ops.linear_swiglu(s1, w_gu, defer=True)
    p2 = ops.linear(h, d["down"], torch.float32, defer=True)
    if last == "plain":
        return x, p2.compute(), s1
    s2 = ops.linear_residual_norm(p2, x, d["nw2"], eps)
    q = ops.linear(s2, d["wq"], torch.bfloat16)
    return x, q, s1


@pytest.mark.parametrize("T,K0,d,F,N2", [(8, 2048, 2048, 8192, 3072), (1, 2048, 2048, 8192, 3072), (3, 264, 200, 320, 136),
                                          (16, 64, 128, 64, 72), (17, 512, 328, 192, 640), (40, 328, 1088, 256, 200),
                                          (64, 2048, 2048, 1024, 3072)])
def test_chain_of_four_products(T, K0, d, F, N2):
    from picolm_b200 import ops
    from picolm_b200.ops import chain
    assert chain.wanted(T)
    eps = 1e-5
    c = _case(T, K0, d, F, N2, T + d + F)
    x2_ref, q_ref, delta_ref = _reference(c, eps)
    x, q, s1 = _run(c, eps)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert isinstance(s1, ops.ScaledRows) and s1.chain is not None and not s1.chain.pending
    assert s1.chain.launched == 1                                     # four products, one launch
    assert torch.allclose(x.double().cpu(), x2_ref, atol=3e-2, rtol=2e-2)
    err = (q.double().cpu() - q_ref).abs().max().item()
    assert err <= 0.06 * max(1.0, q_ref.abs().max().item()), err
    # the chain that ends in a plain product (the last layer: the delta for the final norm)
    x, delta, _ = _run(c, eps, last="plain")
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert delta.dtype == torch.float32
    assert torch.allclose(delta.double().cpu(), delta_ref, atol=3e-2, rtol=2e-2)
    # the same products run one by one give the same within rounding
    old = chain.ENABLED
    chain.ENABLED = False
    try:
        x_1, q_1, s1_1 = _run(c, eps)
        assert s1_1.chain is None
    finally:
        chain.ENABLED = old
    torch.cuda.synchronize()
    assert torch.allclose(x.double().cpu() + delta.double().cpu(), x_1.double().cpu(), atol=2e-2, rtol=1e-2)
    assert (q.float() - q_1.float()).abs().max().item() <= 0.06 * max(1.0, q_ref.abs().max().item())


def test_rows_of_a_chain_do_not_depend_on_their_batch():
    """Row t of a chain's results is the same bits whether it runs alone, among 8 or among 40 rows: how the
    products are dealt out over the SMs depends on their shapes alone, and every sum runs in a fixed order."""
    from picolm_b200 import ops
    eps = 1e-5
    c = _case(40, 512, 328, 192, 640, 5)
    _, q40, _ = _run(c, eps)
    for rows in (slice(0, 8), slice(13, 14), slice(39, 40)):
        sub = {k: (v[rows].contiguous() if k in ("a", "x") else v) for k, v in c.items()}
        x_s, q_s, _ = _run(sub, eps)
        assert torch.equal(q_s, q40[rows])
    ops.check_status(DEV)


def test_chain_inside_the_engine(tmp_path):
    """A decode step at the 1B widths launches one chain per layer boundary, and its logits are those of
    the step without chains, within rounding."""
    from harness import run_batch
    from picolm_b200.engine import Engine
    from picolm_b200.ops import chain
    from test_gpu_schedules import WIDE
    from util import assert_close, make_model_dir, random_tokens
    d = make_model_dir(str(tmp_path / "wide"), WIDE, 23, sharpen=4.0)
    reqs = [random_tokens(n, WIDE["vocab_size"], 70 + n) for n in (40, 9, 25)]
    outs = []
    for on in (True, False):
        old = chain.ENABLED
        chain.ENABLED = on
        try:
            eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 6, max_seqs=4, use_graphs=False)
            before = chain_launches()
            outs.append(torch.cat(run_batch(eng, reqs, [30, 2, 20])))
            assert (chain_launches() > before) == on
        finally:
            chain.ENABLED = old
    assert_close(outs[0], outs[1], "bfloat16", "chains against single launches")


def chain_launches():
    from picolm_b200.ops import chain
    return chain.LAUNCHES[0]
