"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run where the reference checkout is available (it is not shipped with this repository):

    python tests/golden/make_golden.py --reference /path/to/MoC

The script imports the reference's own pure-PyTorch modules (``moc.ffn.MoCSwiGLUFFN`` with
mode "moc" / "moc_gcp" / "moc_2_8" / "moc_post_silu_abs", ``moc.inference.inference_ffn.InferenceMoCSwiGLUFFN``
``masked_reference`` / ``dense_baseline``), runs them on CPU on seeded inputs and writes
``*.npz`` files. bf16 arrays are stored as their uint16 bit patterns (suffix ``__bf16``).

Tie handling: the reference selects with ``torch.topk``, whose choice among equal values is
unspecified. fp32 cases run the reference unmodified (they have no ties at the K-th value;
the script asserts this). bf16 cases are run twice: unmodified (only the multiset of selected
gate values is stored, which does not depend on the tie choice) and with ``torch.topk``
patched to the canonical lowest-index rule, so that the stored outputs are well defined.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from unittest import mock

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle.moc_oracle import canonical_topk, make_inputs  # noqa: E402


def to_np(t: torch.Tensor):
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), True
    return t.numpy(), False


def put(store: dict, name: str, t: torch.Tensor):
    arr, is_bf16 = to_np(t)
    store[name + ("__bf16" if is_bf16 else "")] = arr


class TopkRecorder:
    """Wraps torch.topk: records every call's result; optionally applies the canonical rule."""

    def __init__(self, canonical: bool):
        self.canonical = canonical
        self.calls = []
        self._orig = torch.topk

    def __call__(self, g, k, dim=-1, largest=True, sorted=True):
        if self.canonical:
            vals, idx = canonical_topk(g, k, dim=dim, largest=largest, sorted=sorted)
        else:
            vals, idx = self._orig(g, k, dim=dim, largest=largest, sorted=sorted)
        self.calls.append((g.detach().clone(), vals.detach().clone(), idx.detach().clone()))
        return vals, idx


def run_training_case(ref_ffn, mode, tokens_shape, d, d_ffn, k, dtype, canonical, seed):
    tokens = int(np.prod(tokens_shape))
    x, grad_y, gate_w, up_w, down_w = make_inputs(tokens, d, d_ffn, dtype, seed=seed)
    m = ref_ffn.MoCSwiGLUFFN(d, d_ffn, k, mode=mode).to(dtype)
    with torch.no_grad():
        m.gate_proj.weight.copy_(gate_w)
        m.up_proj.weight.copy_(up_w)
        m.down_proj.weight.copy_(down_w)
    xs = x.reshape(*tokens_shape, d).clone().requires_grad_(True)
    rec = TopkRecorder(canonical)
    with mock.patch("torch.topk", rec):
        y = m(xs)
        y.backward(grad_y.reshape(*tokens_shape, d))
    out = dict(
        y=y.detach().reshape(tokens, d),
        dx=xs.grad.reshape(tokens, d),
        d_gate_w=m.gate_proj.weight.grad,
        d_up_w=m.up_proj.weight.grad,
        d_down_w=m.down_proj.weight.grad,
    )
    return out, rec, m.k_effective


def has_threshold_ties(g, k):
    vals = torch.sort(g.float(), dim=-1, descending=True).values
    return bool((vals[..., k - 1] == vals[..., k]).any()) if k < g.shape[-1] else False


def gen_tiny(ref_ffn, dtype, name):
    store = {}
    shape, d, d_ffn, k = (3, 8), 64, 173, 40
    meta = dict(tokens=24, d=d, d_ffn=d_ffn, k=k, seed=1234)
    for mode in ("moc", "moc_gcp", "moc_2_8", "moc_post_silu_abs"):
        canonical = dtype == torch.bfloat16
        out, rec, k_eff = run_training_case(ref_ffn, mode, shape, d, d_ffn, k, dtype, canonical, seed=1234)
        if dtype == torch.float32 and mode != "moc_2_8":
            g = rec.calls[0][0]
            assert not has_threshold_ties(g.reshape(-1, d_ffn), k), "fp32 case unexpectedly has ties"
        for key, val in out.items():
            put(store, f"{mode}.{key}", val)
        # selected index set per token (sorted), from the recorded topk calls
        if mode == "moc_2_8":
            full = d_ffn // 8
            idx_full = rec.calls[0][2] + (torch.arange(full) * 8).view(1, 1, full, 1)
            parts = [idx_full.reshape(24, -1)]
            if len(rec.calls) > 1:
                parts.append(rec.calls[1][2].reshape(24, -1) + full * 8)
            idx = torch.cat(parts, dim=-1)
        else:
            idx = rec.calls[0][2].reshape(24, -1)
        store[f"{mode}.idx_sorted"] = torch.sort(idx, dim=-1).values.numpy().astype(np.int32)
        store[f"{mode}.k_effective"] = np.int64(k_eff)
        if dtype == torch.bfloat16 and mode == "moc":
            # unmodified torch.topk: tie-independent multiset of selected gate values
            _, rec2, _ = run_training_case(ref_ffn, mode, shape, d, d_ffn, k, dtype, False, seed=1234)
            vals = torch.sort(rec2.calls[0][1].reshape(24, -1).float(), dim=-1).values
            store["moc.unpatched_topk_vals_sorted"] = vals.numpy()
    for key, val in meta.items():
        store["meta." + key] = np.int64(val)
    np.savez_compressed(HERE / f"{name}.npz", **store)
    print("wrote", name, sorted(store)[:4], "...")


def gen_cfg1(ref_ffn):
    """BASELINE config 1: 60m-preset FFN, fp32, X [2,256,512], K=256, reference mode "moc"."""
    store = {}
    shape, d, d_ffn, k = (2, 256), 512, 1376, 256
    out, rec, _ = run_training_case(ref_ffn, "moc", shape, d, d_ffn, k, torch.float32, False, seed=1234)
    assert not has_threshold_ties(rec.calls[0][0].reshape(-1, d_ffn), k)
    rows = np.array([0, 1, 2, 255, 256, 509, 510, 511])
    wrows = np.array([0, 1, 2, 700, 1375])
    store["rows"] = rows
    store["wrows"] = wrows
    store["y_rows"] = out["y"].numpy()[rows]
    store["dx_rows"] = out["dx"].numpy()[rows]
    store["d_gate_w_rows"] = out["d_gate_w"].numpy()[wrows]
    store["d_up_w_rows"] = out["d_up_w"].numpy()[wrows]
    store["d_down_w_cols"] = out["d_down_w"].numpy()[:, wrows]
    for key, val in out.items():
        v = val.double()
        store[f"sum.{key}"] = np.float64(v.sum().item())
        store[f"sumsq.{key}"] = np.float64((v * v).sum().item())
    idx = torch.sort(rec.calls[0][2].reshape(512, -1), dim=-1).values.numpy().astype(np.int16)
    store["idx_sorted_rows"] = idx[rows]
    store["idx_checksum"] = np.int64(idx.astype(np.int64).sum())
    for key, val in dict(tokens=512, d=d, d_ffn=d_ffn, k=k, seed=1234).items():
        store["meta." + key] = np.int64(val)
    np.savez_compressed(HERE / "cfg1_60m_fp32.npz", **store)
    print("wrote cfg1_60m_fp32")


def gen_decode(ref_inf, dtype, name):
    store = {}
    d, d_ffn, k = 64, 176, 40   # d_ffn % 8 == 0 so that the reference's grouped mode accepts it
    for batch in (1, 3):
        x, _, gate_w, up_w, down_w = make_inputs(batch, d, d_ffn, dtype, seed=77 + batch)
        for tag, kwargs in (("global", dict(k=k)), ("g2of8", dict(k=d_ffn * 2 // 8, grouped_a=2, grouped_b=8))):
            m = ref_inf.InferenceMoCSwiGLUFFN(d, d_ffn, **kwargs).to(dtype)
            with torch.no_grad():
                m.gate_proj.weight.copy_(gate_w)
                m.up_proj.weight.copy_(up_w)
                m.down_proj.weight.copy_(down_w)
                rec = TopkRecorder(canonical=True)
                with mock.patch("torch.topk", rec):
                    y = m(x, mode="masked_reference")
                put(store, f"b{batch}.{tag}.masked_reference", y)
                if tag == "global":
                    put(store, f"b{batch}.dense_baseline", m(x, mode="dense_baseline"))
    for key, val in dict(d=d, d_ffn=d_ffn, k=k).items():
        store["meta." + key] = np.int64(val)
    np.savez_compressed(HERE / f"{name}.npz", **store)
    print("wrote", name)


def gen_host(ref_model, ref_config):
    """The reference's LLaMAModel (moc/model.py) on a tiny configuration, fp32, CPU, ffn_type dense and moc:
    full state_dict, inputs, logits, loss and a few gradients, for the host model of moc_b200.host."""
    cfg = ref_config.MoCConfig(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                               vocab_size=97, max_seq_len=16, k=40)
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=gen)
    labels = ids.clone()
    labels[:, 14:] = -100
    store = {"ids": ids.numpy(), "labels": labels.numpy()}
    torch.manual_seed(0)
    base = ref_model.LLaMAModel(cfg, ffn_type="dense")
    state = {k: v.detach().clone() for k, v in base.state_dict().items()}
    for k, v in state.items():
        store["state." + k] = v.numpy()
    for ffn_type in ("dense", "moc"):
        m = ref_model.LLaMAModel(cfg, ffn_type=ffn_type)
        if ffn_type == "moc":
            # build_ffn picks the Triton helper mode, which needs a GPU; the pure-PyTorch mode is the same function
            import moc.ffn as ref_ffn
            for blk in m.blocks:
                blk.ffn = ref_ffn.MoCSwiGLUFFN(cfg.hidden_size, cfg.intermediate_size, cfg.k, mode="moc")
        m.load_state_dict(state)
        rec = TopkRecorder(canonical=False)
        with mock.patch("torch.topk", rec):
            logits, loss = m(ids, labels=labels)
            loss.backward()
        for g, _, _ in rec.calls:
            assert not has_threshold_ties(g.reshape(-1, g.shape[-1]), cfg.k), "fp32 host case has ties"
        store[f"{ffn_type}.logits"] = logits.detach().numpy()
        store[f"{ffn_type}.loss"] = np.float64(loss.item())
        for name in ("tok_emb.weight", "blocks.0.ffn.gate_proj.weight", "blocks.1.ffn.down_proj.weight",
                     "blocks.0.attn.qkv_proj.weight", "lm_head.weight"):
            store[f"{ffn_type}.grad.{name}"] = dict(m.named_parameters())[name].grad.numpy()
    np.savez_compressed(HERE / "host_tiny_fp32.npz", **store)
    print("wrote host_tiny_fp32")


def gen_decoder(reference_dir):
    """The reference's static-cache decoder (benchmarks/inference/benchmark_decode.py:312-362: DecoderModel with
    forward_prompt / forward_step_static) on a tiny configuration, bf16, CPU, with its FFNs evaluated by their
    dense-masking definition (masked_reference, canonical tie rule): state_dict, prompt, the logits and greedy
    token of every decode step and the channel set of every FFN call, for moc_b200.host.GreedyDecoder. Row kinds: dense and global_moc."""
    import importlib.util

    path = Path(reference_dir) / "benchmarks" / "inference" / "benchmark_decode.py"
    spec = importlib.util.spec_from_file_location("ref_benchmark_decode", path)
    bd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bd)
    hidden, inter, heads, vocab, k, layers, max_seq = 256, 1000, 4, 211, 200, 2, 32
    bd.HIDDEN, bd.INTERMEDIATE, bd.NUM_HEADS, bd.VOCAB_SIZE = hidden, inter, heads, vocab
    for kind in ("dense", "global_moc"):
        bd.ROW_SPECS[kind]["k"] = k
    bd.ROW_SPECS["global_moc"]["ffn_mode"] = "masked_reference"      # the CPU-runnable definition of the same row
    store = {}
    for key, val in dict(hidden=hidden, inter=inter, heads=heads, vocab=vocab, k=k, layers=layers, max_seq=max_seq).items():
        store["meta." + key] = np.int64(val)
    gen = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, vocab, (1, 8), generator=torch.Generator().manual_seed(12))
    store["prompt"] = prompt.numpy()
    steps = 6
    state = None
    for kind in ("dense", "global_moc"):
        torch.manual_seed(0)
        model = bd.DecoderModel(layers, kind, "cpu", torch.bfloat16, max_seq).to(torch.bfloat16).eval()
        if state is None:
            with torch.no_grad():
                for p_ in model.parameters():      # matrices ~N(0, 0.05) from seed 11, norm weights stay 1
                    if p_.dim() > 1:
                        p_.copy_(torch.randn(p_.shape, generator=gen) * 0.05)
            state = {k_: v.detach().clone() for k_, v in model.state_dict().items()}
            # the weights are not stored: decoder_weights() below rebuilds them from the seed in this order
            store["state_names"] = np.array([k_ for k_, v in model.named_parameters() if v.dim() > 1])
            store["state_shapes"] = np.array([list(v.shape) for _, v in model.named_parameters() if v.dim() > 1])
        model.load_state_dict(state)
        model.allocate_cache("cpu", torch.bfloat16)
        rec = TopkRecorder(canonical=True)
        with torch.no_grad(), mock.patch("torch.topk", rec):
            logits = model.forward_prompt(prompt)[:, -1]
            tokens, all_logits = [], [logits]
            cur = logits.argmax(dim=-1, keepdim=True)
            for i in range(steps):
                tokens.append(cur)
                logits = model.forward_step_static(cur, torch.tensor(prompt.shape[1] + i))[:, -1]
                all_logits.append(logits)
                cur = logits.argmax(dim=-1, keepdim=True)
        put(store, f"{kind}.logits", torch.stack(all_logits, dim=1))      # [1, steps + 1, vocab]
        # the channel sets the reference selected, in call order (prompt pass: one call per layer over the prompt
        # rows; then one call per layer and decode step), each sorted by channel
        for c, (_, _, idx) in enumerate(rec.calls):
            store[f"{kind}.idx.{c}"] = idx.sort(dim=-1).values.to(torch.int16).numpy()
        store[f"{kind}.tokens"] = torch.cat(tokens, dim=1).numpy()            # [1, steps]: inputs of the decode steps
    np.savez_compressed(HERE / "decoder_tiny_bf16.npz", **store)
    print("wrote decoder_tiny_bf16")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of xiaohuangji/MoC")
    ap.add_argument("--only", default="", help="comma-separated subset: tiny,cfg1,decode,decoder,host (default: all)")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    sys.path.insert(0, args.reference)
    import moc.ffn as ref_ffn  # the reference's own module
    import moc.inference.inference_ffn as ref_inf

    torch.set_num_threads(1)   # fixed reduction order
    if not only or "tiny" in only:
        gen_tiny(ref_ffn, torch.float32, "tiny_fp32")
        gen_tiny(ref_ffn, torch.bfloat16, "tiny_bf16")
    if not only or "cfg1" in only:
        gen_cfg1(ref_ffn)
    if not only or "decode" in only:
        gen_decode(ref_inf, torch.float32, "decode_fp32")
        gen_decode(ref_inf, torch.bfloat16, "decode_bf16")
    if not only or "decoder" in only:
        gen_decoder(args.reference)
    if not only or "host" in only:
        import moc.config as ref_config
        import moc.model as ref_model
        gen_host(ref_model, ref_config)


if __name__ == "__main__":
    main()
