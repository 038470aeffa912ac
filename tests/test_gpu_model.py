"""Drop-in modules (qllm2_b200.model) against outputs of the reference V11LM stored in
tests/golden/model_*.npz: logits, PAM state, fused-CE loss, gradients, greedy decode ids."""
import os

import numpy as np
import pytest
import torch

from qllm2_b200 import model as M
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _load(golden_dir, name):
    g = np.load(os.path.join(golden_dir, f"model_{name}.npz"))
    kw = {}
    for k_, v_ in zip(g["cfg_keys"], g["cfg_vals"]):
        v_ = str(v_)
        kw[str(k_)] = (v_ == "True") if v_ in ("True", "False") else (float(v_) if "." in v_ else int(v_))
    net = M.V11LM(M.V11Config(**kw))
    sd = {k_[6:]: torch.from_numpy(g[k_]) for k_ in g.files if k_.startswith("param:")}
    net.load_state_dict(sd)
    return g, net.to(DEV).eval()


@pytest.mark.parametrize("name", ["k1", "k3", "d64"])
def test_forward_loss_grads_fp32(golden_dir, name):
    g, net = _load(golden_dir, name)
    ids = torch.from_numpy(g["ids"]).to(DEV)
    x = ids[:, :-1]
    with torch.no_grad():
        logits, states, _ = net(x)
    assert_close(logits.cpu().numpy(), g["logits"], 1e-4, "logits")
    assert_close(states[0].cpu().numpy(), g["state0"], 1e-4, "layer-0 PAM state")
    labels = torch.from_numpy(g["labels"]).to(DEV)
    loss, _ = net.fused_ce_loss(x, labels, chunk=32)
    loss.backward()
    ref = float(g["loss"])
    assert abs(float(loss.detach()) - ref) <= 1e-5 * ref, (float(loss.detach()), ref)
    params = dict(net.named_parameters())
    for k_ in g.files:
        if k_.startswith("grad:"):
            assert_close(params[k_[5:]].grad.cpu().numpy(), g[k_], 2e-4, k_)


@pytest.mark.parametrize("name", ["k1", "k3", "d64"])
def test_greedy_decode_ids_exact(golden_dir, name):
    g, net = _load(golden_dir, name)
    prompt = torch.from_numpy(g["ids"][:1, :20]).to(DEV)
    out = net.generate(prompt, max_new_tokens=len(g["greedy"]), temperature=0.0)
    got = out[0, 20:].cpu().numpy()
    if not np.array_equal(got, g["greedy"]):
        first = int(np.argmax(got != g["greedy"]))
        raise AssertionError(f"greedy ids diverge at step {first}: got {got}, want {g['greedy']}, "
                             f"reference top-1/top-2 margin there {g['greedy_margin'][first]:.3e}")


def test_bf16_model_tracks_reference(golden_dir):
    """bf16 weights/activations, d=64: the scan runs on tensor cores; logits within 2e-2 of fp32."""
    g, net = _load(golden_dir, "d64")
    net = net.bfloat16()
    x = torch.from_numpy(g["ids"]).to(DEV)[:, :-1]
    with torch.no_grad():
        logits, _, _ = net(x)
    assert_close(logits.float().cpu().numpy(), g["logits"], 2e-2, "bf16 logits")


def test_autocast_mixed_dtypes_are_unified(golden_dir):
    """Under bf16 autocast RoPE leaves q, k in fp32 while v is bf16: the scan wrapper must bring them to
    one dtype (a mismatch used to be read through q's dtype)."""
    g, net = _load(golden_dir, "k3")
    x = torch.from_numpy(g["ids"]).to(DEV)[:, :-1]
    labels = torch.from_numpy(g["labels"]).to(DEV)
    net.train()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        lm, _, _ = net._hidden_to_lm(x)
    loss = net.ce_from_lm(lm.bfloat16(), labels)
    loss.backward()
    torch.cuda.synchronize()
    ref = float(g["loss"])
    assert abs(float(loss.detach()) - ref) <= 2e-2 * ref
    assert all(torch.isfinite(p.grad).all() for p in net.parameters() if p.grad is not None)
