"""Prefill -> decode sessions for the Qwen2-architecture graphs on the CUDA backend.

The reference extracts two graphs - a prefill graph over a fixed prompt length and a
single-token decode graph over a fixed-shape KV cache - and records which prefill output
feeds which decode input in ``qwen2_kv_mapping.json``
(examples/extract_qwen_ir.py:145-173).  Its driver then downloads every prefill K/V
tensor, pads it to the cache length on the host and uploads it again
(examples/run_qwen.py:132-147).  Here the same mapping format drives a device-side
hand-off: the prefill rows are copied into zero-filled cache buffers by the library's
strided-copy kernel, and the decode loop keeps caches, arg-max and the next token on the
device.
"""

from __future__ import annotations

import ctypes as C
import json
from typing import Any

import numpy as np

FIXED_INPUTS = ("input_ids", "attention_mask", "position_ids", "cache_position")


def _name(spec) -> str:
    return spec["name"] if isinstance(spec, dict) else spec.name


def _ir_part(ir, key: str) -> list:
    return ir[key] if isinstance(ir, dict) else getattr(ir, key)


def kv_mapping(prefill_ir, decode_ir, num_layers: int, prefill_seq_len: int, max_cache_len: int) -> dict:
    """The prefill-output <-> decode-input/output table, in the reference's JSON layout.
    Accepts IR dicts or objects with ``graph_inputs`` / ``graph_outputs`` lists."""
    prefill_kv = _ir_part(prefill_ir, "graph_outputs")[1:]          # [0] is the logits
    decode_in = [s for s in _ir_part(decode_ir, "graph_inputs") if _name(s) not in FIXED_INPUTS]
    decode_out = _ir_part(decode_ir, "graph_outputs")[1:]
    if not (len(prefill_kv) == len(decode_in) == len(decode_out) == 2 * num_layers):
        raise ValueError(f"expected {2 * num_layers} K/V tensors, found {len(prefill_kv)} prefill outputs, "
                         f"{len(decode_in)} decode inputs, {len(decode_out)} decode outputs")
    layers = []
    for i in range(num_layers):
        layers.append({
            "layer": i,
            "prefill_key_output": _name(prefill_kv[2 * i]), "prefill_value_output": _name(prefill_kv[2 * i + 1]),
            "decode_key_input": _name(decode_in[2 * i]), "decode_value_input": _name(decode_in[2 * i + 1]),
            "decode_key_output": _name(decode_out[2 * i]), "decode_value_output": _name(decode_out[2 * i + 1]),
        })
    return {"num_layers": num_layers, "prefill_seq_len": prefill_seq_len, "max_cache_len": max_cache_len, "layers": layers}


def save_kv_mapping(prefill_ir, decode_ir, num_layers: int, prefill_seq_len: int, max_cache_len: int,
                    path: str = "qwen2_kv_mapping.json") -> dict:
    mapping = kv_mapping(prefill_ir, decode_ir, num_layers, prefill_seq_len, max_cache_len)
    with open(path, "w") as f:
        json.dump(mapping, f, indent=2)
    return mapping


def load_kv_mapping(path: str) -> dict:
    with open(path) as f:
        return json.load(f)


def hand_off_kv(prefill_outputs: dict[str, Any], mapping: dict, decode_ir, backend, valid_rows: int | None = None) -> dict[str, Any]:
    """Decode-graph cache buffers filled from prefill outputs, on the device.

    ``prefill_outputs`` maps prefill output names to device buffers ``[B, H, T, D]``; the result
    maps decode input names to new zero-filled buffers ``[B, H, max_cache_len, D]`` whose rows
    ``0..valid_rows`` (default: all T prefill rows) hold the prefill K/V."""
    import torch

    from cuda_runtime import native
    from cuda_runtime.cuda_backend import CUDABuffer

    lib = native.load()
    specs = {_name(s): s for s in _ir_part(decode_ir, "graph_inputs")}
    T = int(mapping["prefill_seq_len"]) if valid_rows is None else int(valid_rows)
    out: dict[str, Any] = {}
    stream = torch.cuda.current_stream().cuda_stream if str(backend.device).startswith("cuda") else 0
    for layer in mapping["layers"]:
        for src_name, dst_name in ((layer["prefill_key_output"], layer["decode_key_input"]),
                                   (layer["prefill_value_output"], layer["decode_value_input"])):
            src = prefill_outputs[src_name]
            src_t = src.native_handle
            spec = specs[dst_name]
            shape = tuple(spec["shape"] if isinstance(spec, dict) else spec.shape)
            B, H, S, D = shape
            if tuple(src_t.shape[:2]) != (B, H) or src_t.shape[3] != D or T > src_t.shape[2] or T > S:
                raise ValueError(f"prefill tensor '{src_name}' {tuple(src_t.shape)} does not fit decode input '{dst_name}' {shape}")
            dst_t = torch.zeros(shape, dtype=src_t.dtype, device=src_t.device)
            if T > 0:
                dt = str(src_t.dtype).replace("torch.", "")
                d = native.make_tensor(dst_t.data_ptr(), dt, (B, H, T, D), (H * S * D, S * D, D, 1))
                s = native.make_tensor(src_t.data_ptr(), dt, (B, H, T, D), tuple(src_t.stride()))
                native.check(lib.b200_strided_copy(C.byref(d), C.byref(s), stream), "KV hand-off")
            out[dst_name] = CUDABuffer(dst_t)
    return out


class QwenSession:
    """Greedy generation with a prefill graph and a decode graph on one GPU.

    ``prefill`` runs the prompt (``[B, T]`` token ids, T = the prefill graph's length) and moves
    its K/V into the decode caches; ``step`` decodes one token for every sequence.  Token ids are
    produced by the device arg-max kernel (lowest index wins ties, like ``torch.argmax`` on the
    reference's CPU path) and only they cross to the host.
    """

    def __init__(self, prefill_ir: dict, decode_ir: dict, weights: dict, num_layers: int, device_id: int = 0):
        from cuda_compiler import compile_subgraph, is_cuda_op_supported
        from cuda_runtime import CUDABackend
        from npu_compiler import partition
        from npu_runtime import DAGExecutor

        self.backend = CUDABackend(device_id)
        self.prefill_ir, self.decode_ir = prefill_ir, decode_ir
        self._pre = DAGExecutor(partition(prefill_ir, is_cuda_op_supported), self.backend, compile_subgraph)
        self._dec = DAGExecutor(partition(decode_ir, is_cuda_op_supported), self.backend, compile_subgraph)
        self._pre.load_weights(weights)
        # the decode graph reuses the buffers the prefill graph uploaded (same state-dict keys)
        shared = {}
        for pid, cache in self._pre._npu_weight_cache.items():
            prog = self._pre.npu_programs[pid]
            for ph, buf in cache.items():
                shared[prog.weight_name_mapping.get(ph, ph)] = buf
        self._dec.load_weights({**weights, **shared})
        p_in = {s["name"]: s for s in prefill_ir["graph_inputs"]}
        d_in = {s["name"]: s for s in decode_ir["graph_inputs"]}
        self.batch, self.prompt_len = p_in["input_ids"]["shape"]
        self.cache_len = d_in["attention_mask"]["shape"][-1]
        self.mask_dtype = d_in["attention_mask"]["dtype"]
        self.vocab = decode_ir["graph_outputs"][0]["shape"][-1]
        self.mapping = kv_mapping(prefill_ir, decode_ir, num_layers, self.prompt_len, self.cache_len)
        self._kv_in = [s["name"] for s in decode_ir["graph_inputs"] if s["name"] not in FIXED_INPUTS]
        self._kv_out = [o["name"] for o in decode_ir["graph_outputs"][1:]]
        self._logits_name = decode_ir["graph_outputs"][0]["name"]
        self._argmax = self._argmax_executor(self.batch, 1)
        self._argmax_prefill = None
        self.kv: dict[str, Any] = {}
        self.position = 0

    def _argmax_executor(self, B: int, T: int):
        from cuda_compiler import compile_subgraph, is_cuda_op_supported
        from npu_compiler import partition
        from npu_runtime import DAGExecutor

        spec = {"name": "logits", "shape": [B, T, self.vocab], "dtype": self.decode_ir["graph_outputs"][0]["dtype"]}
        out = {"name": "token", "shape": [B, T], "dtype": "int64"}
        ir = {"model_name": "greedy", "graph_inputs": [spec], "graph_outputs": [out], "weights": [], "weight_name_mapping": {},
              "nodes": [{"name": "token", "op_type": "aten.argmax.default", "inputs": [spec], "outputs": [out],
                         "attrs": {"dim": -1, "keepdim": False}}]}
        dag = DAGExecutor(partition(ir, is_cuda_op_supported), self.backend, compile_subgraph)
        dag.load_weights({})
        return dag

    @staticmethod
    def _mask(batch: int, q_len: int, kv_len: int, valid: int, dtype: str) -> np.ndarray:
        """Additive mask [B,1,q_len,kv_len]: 0 where key j <= valid + query index, else the dtype's lowest finite value."""
        import ml_dtypes

        np_dt = np.dtype(ml_dtypes.bfloat16) if dtype == "bfloat16" else np.dtype(dtype)
        neg = float(ml_dtypes.finfo(np_dt).min)
        j = np.arange(kv_len)[None, :]
        i = np.arange(q_len)[:, None] + valid
        m = np.where(j <= i, 0.0, neg).astype(np.float32).astype(np_dt)
        return np.ascontiguousarray(np.broadcast_to(m[None, None], (batch, 1, q_len, kv_len)))

    def prefill(self, input_ids: np.ndarray, prompt_len: int | None = None) -> np.ndarray:
        """Run the prompt; returns the first generated token per sequence ``[B, 1]``.  ``prompt_len``
        (<= the graph's length) is the number of real tokens when the ids are right-padded, as the
        reference pads prompts to its fixed prefill length (examples/run_qwen.py:100-118)."""
        B, T = self.batch, self.prompt_len
        n = T if prompt_len is None else int(prompt_len)
        ids = np.ascontiguousarray(input_ids, dtype=np.int64).reshape(B, T)
        feed = {"input_ids": ids, "attention_mask": self._mask(B, T, T, 0, self.mask_dtype),
                "position_ids": np.broadcast_to(np.arange(T, dtype=np.int64)[None], (B, T)).copy(),
                "cache_position": np.arange(T, dtype=np.int64)}
        out = self._pre.execute(feed)
        self.kv = hand_off_kv(out, self.mapping, self.decode_ir, self.backend, valid_rows=n)
        if self._argmax_prefill is None:
            self._argmax_prefill = self._argmax_executor(B, T)
        tokens = self._argmax_prefill.execute({"logits": out[self.prefill_ir["graph_outputs"][0]["name"]]})["token"].to_numpy()
        self.position = n
        return tokens[:, n - 1:n].astype(np.int64)

    def step(self, token_ids: np.ndarray) -> np.ndarray:
        """Decode one token for each sequence at the current position; returns the next ids ``[B, 1]``."""
        if self.position >= self.cache_len:
            raise RuntimeError(f"the KV cache holds {self.cache_len} rows; position {self.position} does not fit")
        B, pos = self.batch, self.position
        feed = {"input_ids": np.ascontiguousarray(token_ids, dtype=np.int64).reshape(B, 1),
                "attention_mask": self._mask(B, 1, self.cache_len, pos, self.mask_dtype),
                "position_ids": np.full((B, 1), pos, np.int64), "cache_position": np.array([pos], np.int64)}
        feed.update(self.kv)
        out = self._dec.execute(feed)
        self.kv = dict(zip(self._kv_in, [out[n] for n in self._kv_out]))
        self.last_logits = out[self._logits_name]
        self.position += 1
        return self._argmax.execute({"logits": self.last_logits})["token"].to_numpy().reshape(B, 1)

    def generate(self, input_ids: np.ndarray, max_new_tokens: int, prompt_len: int | None = None) -> np.ndarray:
        """``[B, max_new_tokens]`` greedy continuation of the prompt."""
        tok = self.prefill(input_ids, prompt_len)
        toks = [tok]
        for _ in range(max_new_tokens - 1):
            tok = self.step(tok)
            toks.append(tok)
        return np.concatenate(toks, axis=1)
