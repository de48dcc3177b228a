"""Writes the golden fixtures in this directory.

Run from the repository root:  python tests/golden/make_golden.py

The reference's CPU path executes IR nodes with PyTorch's ATen kernels; its tests
compare against the eager module (tests/test_dag_executor.py:372-377,
tests/test_e2e_resnet.py:223-229).  The fixtures therefore hold eager-module
outputs for seeded inputs and seeded weights (weights are regenerated from the
seed by model_zoo, not stored), plus the four known-answer graphs of the
reference's tests/test_cpu_fallback.py:36-173.  The oracle must reproduce all of
them; the CUDA path is then compared with the oracle.
"""

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1] / "pytorch-apple_b200"))

import model_zoo as mz  # noqa: E402

TINY_QWEN = dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1, vocab_size=512)


def tiny_qwen(num_layers=2):
    cfg = mz.qwen2_config(num_layers=num_layers, **TINY_QWEN)
    sd = mz.qwen2_weights(cfg, seed=0)
    model = mz.qwen2_model(cfg, device="cpu")
    missing = model.load_state_dict({k[len("model."):]: v for k, v in sd.items() if "rotary" not in k}, strict=False)
    assert not missing.unexpected_keys
    return cfg, sd, model


def bf16_bits(t):
    return t.contiguous().view(torch.uint16).numpy()


def main():
    g = torch.Generator().manual_seed(0)
    # ---- ResNet-18, batch 2, 64x64 -----------------------------------------
    m = mz.resnet(18, seed=0)
    x = torch.randn(2, 3, 64, 64, generator=g)
    with torch.no_grad():
        y = m(x)
    np.savez_compressed(HERE / "resnet18_b2_64.npz", x=x.numpy(), logits=y.numpy())
    # ---- tiny Qwen2 prefill + one decode step ----------------------------------
    cfg, sd, model = tiny_qwen()
    T, S = 24, 40
    ids = torch.randint(0, cfg.vocab_size, (1, T), generator=g)
    with torch.no_grad():
        pre = mz.QwenPrefillWrapper(model)(ids, mz.causal_mask(1, T, T, 0), torch.arange(T)[None], torch.arange(T))
    kv = []
    for t in pre[1:]:
        buf = torch.zeros(1, t.shape[1], S, t.shape[3], dtype=torch.bfloat16)
        buf[:, :, :T] = t
        kv.append(buf)
    nxt = pre[0][:, -1].argmax(-1, keepdim=True)
    with torch.no_grad():
        dec = mz.QwenDecodeWrapper(model, cfg.num_hidden_layers)(nxt, mz.causal_mask(1, 1, S, T), torch.tensor([[T]]),
                                                                  torch.tensor([T]), *kv)
    np.savez_compressed(HERE / "qwen_tiny.npz", ids=ids.numpy(), prefill_logits=bf16_bits(pre[0]),
                        prefill_k0=bf16_bits(pre[1]), next_id=nxt.numpy(), decode_logits=bf16_bits(dec[0]),
                        decode_k0=bf16_bits(dec[1]), T=T, S=S)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
