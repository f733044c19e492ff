"""Makes tests/golden/reference_tiny.safetensors: a tiny random model run through the
reference's OWN Python model code (tools/model_qwen2.py of Destination2020/Paged-Batch-Engine),
with its weights under checkpoint names, the token ids and the logits it returned.

    python tests/golden/make_reference_golden.py --reference /path/to/Paged-Batch-Engine

The reference's Python model anchors the structure of the plain implementation in
tests/plain/plain_qwen2.py: pre-norm placement, q/k/v with bias and o without, grouped
heads, 1/sqrt(head_dim) causal softmax, silu(w1 x) * w3 x, residuals, final norm, tied
head.  It differs from the reference's C++ engine in the rotary pairing (interleaved
here), theta (fixed 1e4) and the always-tied head, so the comparison runs the plain
implementation with interleaved pairing, theta 1e4 and a tied head.  The reference
returns logits for the last position only, hence one forward pass per prefix length.
"""
import argparse
import importlib.util
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Destination2020/Paged-Batch-Engine")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_tiny.safetensors"))
    args = ap.parse_args()
    spec = importlib.util.spec_from_file_location(
        "ref_model_qwen2", os.path.join(args.reference, "tools", "model_qwen2.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    torch.manual_seed(1234)
    margs = ref.ModelArgs(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=61, hidden_dim=48,
                          norm_eps=1e-6, max_seq_len=32)
    model = ref.Transformer(margs).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():        # no silent identities: random biases and gains
            if name.endswith("bias"):
                p.normal_(0.0, 0.3)
            elif "norm" in name:
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
            else:
                p.mul_(6.0)                              # far from uniform attention
    tokens = torch.randint(0, margs.vocab_size, (1, 19))
    rows = []
    with torch.no_grad():
        for n in range(1, tokens.shape[1] + 1):
            rows.append(model(tokens[:, :n])[0, 0])
    out = {"tokens": tokens[0].to(torch.int32), "logits": torch.stack(rows).float()}
    sd = model.state_dict()
    names = {"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight"}
    for i in range(margs.n_layers):
        p, q = f"layers.{i}.", f"model.layers.{i}."
        for a, b in (("wq", "q_proj"), ("wk", "k_proj"), ("wv", "v_proj")):
            names[p + f"attention.{a}.weight"] = q + f"self_attn.{b}.weight"
            names[p + f"attention.{a}.bias"] = q + f"self_attn.{b}.bias"
        names[p + "attention.wo.weight"] = q + "self_attn.o_proj.weight"
        names[p + "feed_forward.w1.weight"] = q + "mlp.gate_proj.weight"
        names[p + "feed_forward.w2.weight"] = q + "mlp.down_proj.weight"
        names[p + "feed_forward.w3.weight"] = q + "mlp.up_proj.weight"
        names[p + "attention_norm.weight"] = q + "input_layernorm.weight"
        names[p + "ffn_norm.weight"] = q + "post_attention_layernorm.weight"
    for k, v in names.items():
        out[v] = sd[k].detach().float().contiguous().clone()
    from safetensors.torch import save_file
    save_file(out, args.out, metadata={"made_by": "tests/golden/make_reference_golden.py",
                                       "dim": "32", "n_layers": "2", "n_heads": "4", "n_kv_heads": "2",
                                       "hidden_dim": "48", "vocab_size": "61", "norm_eps": "1e-6"})
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    sys.exit(main())
