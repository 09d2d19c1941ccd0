#!/usr/bin/env python
"""Builds ``tests/golden/glm_anchor_{1,2}.npz`` from the reference's vendored goldens.

    python tests/golden/make_glm_anchor_fixtures.py [path-to-reference-checkout]

The reference keeps two captures of a real (toy-width) GLM-MoE-DSA model run, produced by its
``crates/oracles/tests/glm_anchor_driver.py`` from HF transformers and checked by
``crates/oracles/tests/glm_anchor.rs``: ``crates/oracles/tests/glm-anchor-{1,2}.bin``. This script

* reads that container (``crates/oracles/src/golden.rs:143-162,230-247,355-374``: magic ``RIVGMGLD``, a
  list of metadata strings, then named f32 and named i64 tensors, every length a little-endian u64);
* keeps the tensors of the decode KV-cache path: per step ``t`` and layer ``L`` the latent rows, the roped
  keys, the last query row and its attention output, the selection mask and indices, and what the indexer of
  a full layer reads;
* regenerates the model weights this path needs - ``kv_b_proj`` of every layer and the indexer's ``wq_b``,
  ``wk``, ``k_norm``, ``weights_proj`` of the full layers - from the driver's rule: a parameter is a pure
  function of its NAME, ``sha256("<salt>/<name>")`` seeding a torch CPU generator whose ``uniform_`` fills it
  (``glm_anchor_driver.py:96-140``). Whether this image's torch reproduces the draws is CHECKED here, not
  assumed: the prompt ids must regenerate, and the captured attention output of every layer must follow from
  the captured inputs and the regenerated ``kv_b_proj`` in the non-absorbed form the capture was made in;
* writes everything as one small ``.npz`` per golden, which is what the tests read (the reference checkout does
  not travel with the repository).
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def read_golden(path):
    b = open(path, "rb").read()
    o = [8]

    def u64():
        v = struct.unpack_from("<Q", b, o[0])[0]
        o[0] += 8
        return v

    def text():
        n = u64()
        s = b[o[0]:o[0] + n].decode()
        o[0] += n
        return s

    assert b[:8] == b"RIVGMGLD", b[:8]
    meta = dict((text(), text()) for _ in range(u64()))

    def tensors(dt):
        out = {}
        for _ in range(u64()):
            name = text()
            shape = [u64() for _ in range(u64())]
            n = u64()
            out[name] = np.frombuffer(b, dtype=dt, count=n, offset=o[0]).reshape(shape).copy()
            o[0] += n * out[name].itemsize
        return out

    floats, ints = tensors("<f4"), tensors("<i8")
    assert o[0] == len(b), "trailing bytes"
    return meta, floats, ints


def draw(salt, name, shape):
    """A parameter by the driver's rule (glm_anchor_driver.py:101-118)."""
    import torch
    h = hashlib.sha256(f"{salt}/{name}".encode()).digest()
    g = torch.Generator().manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    flat = torch.empty(int(np.prod(shape)), dtype=torch.float32)
    leaf = name.rsplit(".", 2)[-2] if "." in name else name
    if name.endswith(".bias"):
        flat.uniform_(-0.05, 0.05, generator=g)
    elif "norm" in leaf:
        flat.uniform_(0.8, 1.2, generator=g)
    else:
        flat.uniform_(-0.08, 0.08, generator=g)
    return flat.view(*shape).numpy().copy()


def convert(src, dst):
    import torch
    meta, F, I = read_golden(src)
    cfg, salt = json.loads(meta["config"]), meta["salt"]
    H, nope, rope, vh, kvl = (cfg[k] for k in ("num_attention_heads", "qk_nope_head_dim", "qk_rope_head_dim",
                                                "v_head_dim", "kv_lora_rank"))
    nh, hd, hidden, qlr = cfg["index_n_heads"], cfg["index_head_dim"], cfg["hidden_size"], cfg["q_lora_rank"]
    layers, steps = cfg["num_hidden_layers"], int(meta["decode_steps"]) + 1
    full = I["structure.indexer_is_full"]
    out = {"meta_json": np.array(json.dumps(meta)), "prompt_ids": I["prompt.ids"], "indexer_is_full": full}

    # 1. does this torch reproduce the driver's draws?
    h = hashlib.sha256(f"{salt}/prompt".encode()).digest()
    g = torch.Generator().manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    ids = torch.randint(0, cfg["vocab_size"], (1, I["prompt.ids"].size), generator=g).numpy().ravel()
    assert np.array_equal(ids, I["prompt.ids"]), "this torch does not reproduce the driver's generator"

    for L in range(layers):
        w = draw(salt, f"model.layers.{L}.self_attn.kv_b_proj.weight", (H * (nope + vh), kvl))
        out[f"L{L}.kv_b_proj"] = w
        if full[L]:
            pre = f"model.layers.{L}.self_attn.indexer."
            out[f"L{L}.index.wq_b"] = draw(salt, pre + "wq_b.weight", (nh * hd, qlr))
            out[f"L{L}.index.wk"] = draw(salt, pre + "wk.weight", (hd, hidden))
            out[f"L{L}.index.k_norm.weight"] = draw(salt, pre + "k_norm.weight", (hd,))
            out[f"L{L}.index.k_norm.bias"] = draw(salt, pre + "k_norm.bias", (hd,))
            out[f"L{L}.index.weights_proj"] = draw(salt, pre + "weights_proj.weight", (nh, hidden))
        # 2. the regenerated kv_b_proj must explain the captured attention (non-absorbed form, f64)
        W = w.astype(np.float64).reshape(H, nope + vh, kvl)
        q = F[f"t0.L{L}.attend.q"][0, :, -1].astype(np.float64)
        c = F[f"t0.L{L}.kv_latent"][0].astype(np.float64)
        kpe = F[f"t0.L{L}.attn.k.post_rope"][0, 0].astype(np.float64)
        mask = F[f"t0.L{L}.attend.mask_last_row"].astype(np.float64)
        want = F[f"t0.L{L}.attend.out"][0, -1].astype(np.float64)
        for hh in range(H):
            s = ((c @ W[hh, :nope].T) @ q[hh, :nope] + kpe @ q[hh, nope:]) * (nope + rope) ** -0.5 + mask
            p = np.exp(s - s.max())
            got = (p / p.sum()) @ (c @ W[hh, nope:].T)
            assert np.abs(got - want[hh]).max() < 1e-6, ("kv_b_proj does not regenerate", L, hh)
        for t in range(steps):
            p_ = f"t{t}.L{L}."
            out[p_ + "kv_latent"] = F[p_ + "kv_latent"][0]                       # [S, kvl] rows this step adds
            out[p_ + "k_rope"] = F[p_ + "attn.k.post_rope"][0, 0]                 # [S, rope]
            out[p_ + "q_last"] = F[p_ + "attend.q"][0, :, -1]                      # [H, nope + rope]
            out[p_ + "out_last"] = F[p_ + "attend.out"][0, -1]                     # [H, vh]
            out[p_ + "mask_last_row"] = F[p_ + "attend.mask_last_row"]             # [T] 0 / -inf
            out[p_ + "topk_indices"] = I[p_ + "topk_indices"]
            if full[L]:
                out[p_ + "hidden"] = F[p_ + "norm.in"][0]                          # [S, hidden] the layer's normed input
                out[p_ + "q_resid"] = F[p_ + "q_resid"][0]                          # [S, q_lora]
                out[p_ + "index.q_rope"] = F[p_ + "index.q.post_rope"][0]           # [S, nh, rope]
                out[p_ + "index.k_rope"] = F[p_ + "index.k.post_rope"][0, :, 0]     # [S, rope]
    out["torch_version_used_for_weights"] = np.array(torch.__version__)
    np.savez_compressed(dst, **out)
    print(f"{os.path.basename(dst)}: {len(out)} arrays, {os.path.getsize(dst)} bytes; weights regenerate with torch "
          f"{torch.__version__} (prompt ids and all {layers} kv_b_proj checks passed)")


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    for n in (1, 2):
        convert(os.path.join(ref, "crates/oracles/tests", f"glm-anchor-{n}.bin"), os.path.join(HERE, f"glm_anchor_{n}.npz"))
