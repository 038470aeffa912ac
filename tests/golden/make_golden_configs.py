"""Golden fixtures at the configured model sizes: run the REFERENCE V11LM (random init from
torch.manual_seed(0)) and store what a test on a machine without the reference needs.

  train_c3.npz   8-block v11_e3_k3_chat model (dim 384, H 6, d 64, K 3, chunk 64, vocab 50261), the first two
                 rows of the seeded [8, 2049] id matrix, T = 2048: loss under CPU bf16 autocast and in plain
                 fp32, norms and leading samples of a handful of parameter gradients (both runs).
  decode_c5.npz  12-block dim-768 H 12 d 64 K 3 model, weights rounded to bf16, arithmetic in fp32:
                 prefill + greedy recurrent steps (v11/bench_infer.py:167-193 pattern) for a seeded subset of
                 short prompts; ids, top-1/top-2 margins, top-2 ids of every step.

Weights are not stored (they are reproducible from the seed); checksums of a few parameters are, so a
test can assert that its own construction order drew the same numbers.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_configs.py /path/to/qllm2 [c3|c5]
"""
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/qllm2 [c3|c5]")
REF = sys.argv[1]
WHICH = sys.argv[2:] or ["c3", "c5"]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from v11 import triton_kernels  # noqa: E402
from v11.model import V11Config, V11LM, get_config  # noqa: E402

triton_kernels.set_triton_enabled(False)
torch.set_num_threads(os.cpu_count())

CHECK_PARAMS = ("embed.embed_real.weight", "blocks.0.pam.qkv_proj.weight_real", "blocks.0.cgu.up_proj.weight_imag",
                "lm_head_proj.weight_real")


def checksums(model, names):
    sd = model.state_dict()
    out = {}
    for n_ in names:
        t = sd[n_].double()
        out["check:" + n_] = np.array([float(t.sum()), float(t.abs().sum())])
    return out


def make_c3():
    torch.manual_seed(0)
    cfg = get_config("v11_e3_k3_chat")
    cfg.n_layers, cfg.chunk_size, cfg.dropout, cfg.gradient_checkpointing = 8, 64, 0.0, False
    model = V11LM(cfg).train()
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (8, 2049), generator=gen)[:2]
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    grads_of = ("embed.embed_real.weight", "blocks.0.pam.qkv_proj.weight_real", "blocks.3.pam.dt_proj.weight",
                "blocks.7.pam.o_proj.weight_imag", "blocks.4.cgu.up_proj.weight_real", "lm_head_proj.weight_real",
                "blocks.0.pam.phase_proj.weight", "blocks.5.pam.protect_gate.weight")
    out = {"ids": ids.numpy(), "grads_of": np.array(grads_of)}
    out.update(checksums(model, CHECK_PARAMS))
    params = dict(model.named_parameters())
    for tag, ctx in (("bf16", lambda: torch.autocast("cpu", dtype=torch.bfloat16)), ("fp32", None)):
        model.zero_grad(set_to_none=True)
        t0 = time.time()
        if ctx is not None:
            with ctx():
                lm, _, _ = model._hidden_to_lm(x)
        else:
            lm, _, _ = model._hidden_to_lm(x)
        loss = model.ce_from_lm(lm, y)
        loss.backward()
        out[f"loss_{tag}"] = np.array(float(loss.detach()))
        for n_ in grads_of:
            g = params[n_].grad.detach().float()
            out[f"gnorm_{tag}:{n_}"] = np.array(float(g.double().norm()))
            out[f"ghead_{tag}:{n_}"] = g.reshape(-1)[:256].numpy().copy()
            # rows that certainly carry signal: for the embedding, the rows of the first few input ids
            if n_ == "embed.embed_real.weight":
                out[f"grows_{tag}:{n_}"] = g[ids[0, :8]].numpy().copy()
        print(f"c3 {tag}: loss {float(loss.detach()):.6f} in {time.time() - t0:.0f} s", flush=True)
    path = os.path.join(HERE, "train_c3.npz")
    np.savez_compressed(path, **out)
    print("train_c3", f"{os.path.getsize(path) / 1024:.0f} KiB")


def make_c5(n_prompts=8, lo=32, hi=256, new_tokens=16):
    torch.manual_seed(0)
    cfg = V11Config(vocab_size=50261, dim=768, n_heads=12, head_dim=64, n_layers=12, n_states=3,
                    gate_content_aware=True, dropout=0.0, gradient_checkpointing=False, max_seq_len=8192)
    model = V11LM(cfg)
    out = {}
    out.update(checksums(model, CHECK_PARAMS))
    model = model.bfloat16().float().eval()          # bf16-rounded weights, fp32 arithmetic
    gen = torch.Generator().manual_seed(5)
    lengths = torch.randint(lo, hi + 1, (n_prompts,), generator=gen)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=gen) for n in lengths]
    all_ids, all_margin, all_top2 = [], [], []
    with torch.no_grad():
        for i, p_ in enumerate(prompts):
            t0 = time.time()
            logits, states, _ = model(p_[None])
            step = p_.numel()
            toks, margins, top2 = [], [], []
            for _ in range(new_tokens):
                last = logits[:, -1]
                tk = last.topk(2)
                margins.append(float(tk.values[0, 0] - tk.values[0, 1]))
                top2.append(tk.indices[0].numpy().copy())
                nxt = last.argmax(dim=-1, keepdim=True)
                toks.append(int(nxt))
                logits, states, _ = model(nxt, states=states, step_offset=step)
                step += 1
            all_ids.append(toks)
            all_margin.append(margins)
            all_top2.append(np.stack(top2))
            print(f"c5 prompt {i} len {p_.numel()}: min margin {min(margins):.3e}, {time.time() - t0:.0f} s", flush=True)
    out["prompt_lengths"] = lengths.numpy()
    out["prompt_ids"] = torch.cat(prompts).numpy()
    out["greedy"] = np.array(all_ids)
    out["margin"] = np.array(all_margin)
    out["top2"] = np.stack(all_top2)
    path = os.path.join(HERE, "decode_c5.npz")
    np.savez_compressed(path, **out)
    print("decode_c5", f"{os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    if "c5" in WHICH:
        make_c5()
    if "c3" in WHICH:
        make_c3()
