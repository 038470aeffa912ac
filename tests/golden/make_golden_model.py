"""Model-level golden fixtures: run the REFERENCE V11LM (tiny random-init configurations) and store
its parameters, inputs and outputs, so the drop-in modules can be checked on machines where the
reference is absent.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_model.py /path/to/qllm2
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/qllm2   (a checkout of the reference)")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from v11 import triton_kernels  # noqa: E402
from v11.model import V11Config, V11LM  # noqa: E402

triton_kernels.set_triton_enabled(False)

CONFIGS = {
    "k1": dict(vocab_size=97, dim=32, n_heads=2, head_dim=16, n_layers=2, expand=2, dropout=0.0, max_seq_len=128,
               chunk_size=24, gradient_checkpointing=False),
    "k3": dict(vocab_size=97, dim=32, n_heads=2, head_dim=16, n_layers=2, expand=2, dropout=0.0, max_seq_len=128,
               chunk_size=24, gradient_checkpointing=False, n_states=3, gate_content_aware=True),
    "d64": dict(vocab_size=131, dim=64, n_heads=1, head_dim=64, n_layers=1, expand=2, dropout=0.0, max_seq_len=256,
                chunk_size=64, gradient_checkpointing=False),
}


def make(name, kw, T=50, new_tokens=12):
    torch.manual_seed(0)
    cfg = V11Config(**kw)
    model = V11LM(cfg)
    # move the zero-initialised routing / gate weights off zero so that every path carries signal
    gen = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n_, p in model.named_parameters():
            if "phase_proj" in n_ or "dt_proj.weight" in n_ or "protect_gate.weight" in n_:
                p.add_(torch.randn(p.shape, generator=gen) * 0.3)
    model.eval()
    ids = torch.randint(0, cfg.vocab_size, (2, T + 1), generator=gen)
    x, y = ids[:, :-1], ids[:, 1:]
    out = {"cfg_keys": np.array(list(kw.keys())), "cfg_vals": np.array([str(v) for v in kw.values()]), "ids": ids.numpy()}
    for k_, v_ in model.state_dict().items():
        out["param:" + k_] = v_.numpy()
    with torch.no_grad():
        logits, states, _ = model(x)
    out["logits"] = logits.numpy()
    out["state0"] = states[0].numpy()
    labels = y.clone()
    labels[:, ::9] = -100
    loss, _ = model.fused_ce_loss(x, labels, chunk=32)
    loss.backward()
    out["loss"] = loss.detach().numpy()
    out["labels"] = labels.numpy()
    for k_ in ("embed.embed_real.weight", "blocks.0.pam.dt_proj.weight", "blocks.0.pam.qkv_proj.weight_real",
               "blocks.1.pam.phase_proj.weight" if kw.get("n_states", 1) > 1 else "blocks.0.cgu.up_proj.weight_imag",
               "lm_head_proj.weight_real"):
        if dict(model.named_parameters()).get(k_) is not None:
            out["grad:" + k_] = dict(model.named_parameters())[k_].grad.numpy()
    # greedy decode: prefill then recurrent steps (v11/bench_infer.py:173-190 pattern), batch of 1
    with torch.no_grad():
        prompt = x[:1, :20]
        logits, states, _ = model(prompt)
        step = prompt.shape[1]
        toks, margins, step_logits = [], [], []
        for _ in range(new_tokens):
            last = logits[:, -1]
            step_logits.append(last[0].numpy())
            top2 = last.topk(2).values[0]
            margins.append(float(top2[0] - top2[1]))
            nxt = last.argmax(dim=-1, keepdim=True)
            toks.append(int(nxt))
            logits, states, _ = model(nxt, states=states, step_offset=step)
            step += 1
    out["greedy"] = np.array(toks)
    out["greedy_margin"] = np.array(margins)
    out["greedy_logits"] = np.stack(step_logits)
    path = os.path.join(HERE, f"model_{name}.npz")
    np.savez_compressed(path, **out)
    print(name, f"{os.path.getsize(path) / 1024:.0f} KiB", "loss", float(loss), "min margin", min(margins))


if __name__ == "__main__":
    for name, kw in CONFIGS.items():
        make(name, kw)
