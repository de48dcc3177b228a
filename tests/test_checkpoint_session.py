"""Checkpoint loading and prefill -> decode sessions (host logic; the library is replaced by
the torch stand-in).  Loader semantics follow the reference's examples/run_qwen_graph.py:25-82
and examples/hf_utils.py:18-140; the KV mapping follows examples/extract_qwen_ir.py:145-173."""

import json

import numpy as np
import pytest
import torch

import model_zoo as mz
from helpers import to_f32
from ir_export import extract_ir
from oracle.ir_interpreter import IRInterpreter


def _tiny():
    from golden.make_golden import tiny_qwen

    return tiny_qwen()


def test_safetensors_round_trip_keeps_bits(tmp_path):
    import ml_dtypes

    from checkpoint import read_safetensors, write_safetensors

    rng = np.random.RandomState(0)
    tensors = {"a.weight": rng.randn(5, 7).astype(np.float32).astype(ml_dtypes.bfloat16), "b": rng.randn(3).astype(np.float32),
               "ids": np.arange(6, dtype=np.int64).reshape(2, 3), "h": rng.randn(4, 2).astype(np.float16), "empty": np.zeros((0,), np.float32)}
    write_safetensors(tmp_path / "m.safetensors", tensors, {"format": "pt"})
    back = read_safetensors(tmp_path / "m.safetensors")
    assert set(back) == set(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape
        np.testing.assert_array_equal(back[k].view(np.uint8), np.ascontiguousarray(v).view(np.uint8))
    # the container is the published one: the safetensors package reads the same tensors
    st = pytest.importorskip("safetensors.torch")
    ref = st.load_file(str(tmp_path / "m.safetensors"))
    assert ref["a.weight"].dtype == torch.bfloat16
    np.testing.assert_array_equal(ref["a.weight"].view(torch.uint16).numpy(), tensors["a.weight"].view(np.uint16))
    with open(tmp_path / "bad.safetensors", "wb") as f:
        f.write(b"\xff" * 8 + b"{}")
    with pytest.raises(ValueError):
        read_safetensors(tmp_path / "bad.safetensors")


def test_load_numpy_weights_prefix_tied_head_inv_freq_and_shards(tmp_path):
    """Checkpoint keys have no wrapper prefix, the head is tied (not stored), inv_freq is not stored,
    tensors are spread over two shards with an index."""
    import ml_dtypes

    from checkpoint import load_numpy_weights, write_safetensors

    cfg, sd, model = _tiny()
    ir = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, 8, None, device="cpu"), "p")
    npw = mz.state_dict_numpy(sd)
    stored = {k[len("model."):]: v for k, v in npw.items() if "inv_freq" not in k and "lm_head" not in k}   # "model.model.x" -> "model.x"
    keys = sorted(stored)
    shards = {"model-00001-of-00002.safetensors": keys[: len(keys) // 2], "model-00002-of-00002.safetensors": keys[len(keys) // 2:]}
    for fname, ks in shards.items():
        write_safetensors(tmp_path / fname, {k: stored[k] for k in ks})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: f for f, ks in shards.items() for k in ks}}))
    (tmp_path / "config.json").write_text(json.dumps({"rope_theta": 1e6}))
    got = load_numpy_weights(tmp_path, ir)
    need = {w["name"] for w in ir["weights"]}
    assert need <= set(got)
    for k in need:
        if "inv_freq" in k:
            np.testing.assert_allclose(got[k], npw[k], rtol=1e-6)
            assert got[k].dtype == np.float32
        elif "lifted_tensor" in k:
            assert got[k].shape == (0,)     # the prefill graph's empty initial cache
        else:
            assert got[k].dtype == np.dtype(ml_dtypes.bfloat16)
            np.testing.assert_array_equal(got[k].view(np.uint16), npw[k].view(np.uint16))
    head = next(k for k in need if "lm_head.weight" in k)
    np.testing.assert_array_equal(got[head].view(np.uint16), npw["model.model.embed_tokens.weight"].view(np.uint16))
    # without a config the reference's base of 10000 is used
    (tmp_path / "config.json").unlink()
    inv = load_numpy_weights(tmp_path, ir)[next(k for k in need if "inv_freq" in k)]
    np.testing.assert_allclose(inv, 1.0 / (10000.0 ** (np.arange(64, dtype=np.float32) / 64)), rtol=1e-6)
    # an fp32 checkpoint is narrowed to the compute dtype
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {k: stored[k].astype(np.float32) for k in shards["model-00001-of-00002.safetensors"]})
    again = load_numpy_weights(tmp_path, ir)
    k0 = "model." + shards["model-00001-of-00002.safetensors"][0]
    assert again[k0].dtype == np.dtype(ml_dtypes.bfloat16)
    np.testing.assert_array_equal(again[k0].view(np.uint16), npw[k0].view(np.uint16))


def test_kv_mapping_has_the_reference_layout(tmp_path):
    from qwen_session import kv_mapping, load_kv_mapping, save_kv_mapping

    cfg, sd, model = _tiny()
    L = cfg.num_hidden_layers
    irp = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, 1, 8, None, device="cpu"), "p")
    ird = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, 1, 1, 32, device="cpu"), "d")
    m = save_kv_mapping(irp, ird, L, 8, 32, str(tmp_path / "qwen2_kv_mapping.json"))
    assert m == load_kv_mapping(str(tmp_path / "qwen2_kv_mapping.json")) == kv_mapping(irp, ird, L, 8, 32)
    assert set(m) == {"num_layers", "prefill_seq_len", "max_cache_len", "layers"} and len(m["layers"]) == L
    assert set(m["layers"][0]) == {"layer", "prefill_key_output", "prefill_value_output", "decode_key_input", "decode_value_input",
                                   "decode_key_output", "decode_value_output"}
    assert m["layers"][1]["prefill_key_output"] == irp["graph_outputs"][3]["name"]
    assert m["layers"][1]["decode_value_input"] == ird["graph_inputs"][4 + 3]["name"]
    assert m["layers"][1]["decode_value_output"] == ird["graph_outputs"][1 + 3]["name"]
    with pytest.raises(ValueError):
        kv_mapping(irp, ird, L + 1, 8, 32)


def test_session_prefill_hand_off_and_greedy_decode_match_the_oracle(fake_native):
    """Tokens of a whole session (prompt right-padded to the prefill graph's length) equal the
    oracle's greedy tokens; the hand-off puts the prefill rows at the start of zero-filled caches."""
    from qwen_session import QwenSession

    cfg, sd, model = _tiny()
    L, T, S, B, n_real, new = cfg.num_hidden_layers, 16, 40, 2, 11, 5
    irp = extract_ir(mz.QwenPrefillWrapper(model), mz.qwen2_example_inputs(cfg, B, T, None, device="cpu"), "p")
    ird = extract_ir(mz.QwenDecodeWrapper(model, L), mz.qwen2_example_inputs(cfg, B, 1, S, device="cpu"), "d")
    sess = QwenSession(irp, ird, mz.state_dict_numpy(sd), L)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    ids[:, n_real:] = 0                                             # padding
    got = sess.generate(ids.numpy(), new, prompt_len=n_real)
    assert got.shape == (B, new) and sess.position == n_real + new - 1
    # oracle: the same protocol on the host
    pre = IRInterpreter(irp, sd).execute((ids, mz.causal_mask(B, T, T, 0), torch.arange(T)[None].expand(B, T), torch.arange(T)))
    pn = [o["name"] for o in irp["graph_outputs"]]
    tok = pre[pn[0]][:, n_real - 1].float().argmax(-1, keepdim=True)
    want = [tok]
    kv = []
    for n in pn[1:]:
        buf = torch.zeros(B, pre[n].shape[1], S, pre[n].shape[3], dtype=torch.bfloat16)
        buf[:, :, :n_real] = pre[n][:, :, :n_real]
        kv.append(buf)
    interp = IRInterpreter(ird, sd)
    dn = [o["name"] for o in ird["graph_outputs"]]
    for i in range(new - 1):
        pos = n_real + i
        out = interp.execute((tok, mz.causal_mask(B, 1, S, pos), torch.full((B, 1), pos), torch.tensor([pos]), *kv))
        tok = out[dn[0]][:, -1].float().argmax(-1, keepdim=True)
        kv = [out[n] for n in dn[1:]]
        want.append(tok)
    want = torch.cat(want, 1).numpy()
    if not (got == want).all():   # bf16 rounding may flip a near-tie; then the logits must be that close
        lg = to_f32(sess.last_logits)[:, 0]
        assert np.abs(lg - out[dn[0]][:, 0].float().numpy()).max() < 0.1
        assert (got[:, 0] == want[:, 0]).all()
    else:
        np.testing.assert_array_equal(got, want)
    k0 = sess.kv[sess._kv_in[0]].to_numpy()
    assert k0.shape == (B, 1, S, 128) and (k0.view(np.uint16)[:, :, sess.position:] == 0).all()
