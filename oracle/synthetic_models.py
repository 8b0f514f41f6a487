"""Random-weight model files with the reference engine's tensor names and shapes (TEST INFRASTRUCTURE).

    python oracle/synthetic_models.py DIR [--seed N]

The reference's engine (engine/src/engine.h:229-270, Engine::load) reads three .safetensors files from its models
directory before it answers a request; none of them can be downloaded here. For the protocol-level test (the reference's
own engine built on Linux, once over its own kernels and once over this repository's library) the values do not matter,
only that both builds read the same files, so this script writes files of the same architecture with seeded random
weights:

  anima-base-v1.0.safetensors   the DiT the loader expects (engine/src/dit.cu:11-96: 28 blocks, 2048 wide, adaLN-LoRA
                                rank 256, 6-block LLM adapter, 1024 wide), bf16, about 4 GB
  qwen_3_06b_base.safetensors   the text encoder's layout (engine/src/te.cu:6-28; the loader counts the layers it finds
                                and reads the MLP width from the file: two layers, a shortened vocabulary)
  loras/style_a, style_b        two LoRA files in the naming the engine's loader pairs up (engine/src/engine.h:136-170)
  qwen_image_vae.safetensors    the VAE's layout (engine/src/vae.cu:38-112: channel counts are read from the file; the
                                real ones are used: 96/192/384/384, 16 latent channels)

Weights are uniform with variance gain^2 / fan_in, norm scales 1 +- 0.1, biases small, all stored as bf16. The values
come from one seeded pool that is sliced at rotating offsets, so that writing the files takes seconds, not minutes.
"""
import json
import os
import struct
import sys

import numpy as np

D, AD, FF = 2048, 1024, 8192
TE_VOCAB, T5_VOCAB = 65536, 32768        # token ids in test requests and in the engine's --bench prompt (main.cpp:79-80) stay below these
POOL = 1 << 24


def _bf16(x):
    """float32 array -> bf16 bit patterns (round to nearest even)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class _Writer:
    """One .safetensors file: 8-byte header length, JSON header, tensors back to back (bf16)."""

    layout_only = False     # True (set by write_all(..., layout_only=True)): headers and sizes only, for loader checks on the CPU

    def __init__(self, seed):
        rng = np.random.default_rng(seed)
        self.unit = rng.uniform(-1.0, 1.0, POOL).astype(np.float32)   # the pool, unit scale
        self.scaled = {}                                                 # scale -> bf16 pool
        self.at = 0
        self.entries = []

    def _take(self, n, scale, offset=0.0):
        if self.layout_only:
            return 2 * n                                  # bytes only
        key = (round(float(scale), 9), offset)
        if key not in self.scaled:
            self.scaled[key] = _bf16(self.unit * np.float32(scale) + np.float32(offset))
        pool = self.scaled[key]
        start = (self.at * 7919) % (POOL - 1)
        self.at += 1
        out = np.empty(n, dtype=np.uint16)
        done = 0
        while done < n:
            m = min(n - done, POOL - start)
            out[done:done + m] = pool[start:start + m]
            done += m
            start = 0
        return out

    def weight(self, name, shape, gain=1.0, fan_in=None):
        n = int(np.prod(shape))
        fan = fan_in if fan_in else int(np.prod(shape[1:])) if len(shape) > 1 else 1
        self.entries.append((name, list(shape), self._take(n, gain * np.sqrt(3.0 / fan))))

    def norm(self, name, shape):
        self.entries.append((name, list(shape), self._take(int(np.prod(shape)), 0.1, 1.0)))

    def bias(self, name, n):
        self.entries.append((name, [n], self._take(n, 0.02)))

    def save(self, path):
        header, off = {}, 0
        for name, shape, data in self.entries:
            nbytes = data if isinstance(data, int) else data.nbytes
            header[name] = {"dtype": "BF16", "shape": shape, "data_offsets": [off, off + nbytes]}
            off += nbytes
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * (-len(blob) % 8)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            if self.layout_only:
                f.truncate(8 + len(blob) + off)          # a sparse file: the right names, shapes and size, all-zero values
            else:
                for _, _, data in self.entries:
                    f.write(data.tobytes())
        return off


def write_dit(path, seed=1, blocks=28):
    w = _Writer(seed)
    for i in range(blocks):
        p = "net.blocks.%d." % i
        for a in ("self_attn", "cross_attn"):
            kv_in = D if a == "self_attn" else AD
            w.weight(p + a + ".q_proj.weight", (D, D))
            w.weight(p + a + ".k_proj.weight", (D, kv_in))
            w.weight(p + a + ".v_proj.weight", (D, kv_in))
            w.weight(p + a + ".output_proj.weight", (D, D))
            w.norm(p + a + ".q_norm.weight", (128,))
            w.norm(p + a + ".k_norm.weight", (128,))
        w.weight(p + "mlp.layer1.weight", (FF, D))
        w.weight(p + "mlp.layer2.weight", (D, FF))
        for m in ("self_attn", "cross_attn", "mlp"):
            w.weight(p + "adaln_modulation_%s.1.weight" % m, (256, D))
            w.weight(p + "adaln_modulation_%s.2.weight" % m, (3 * D, 256), gain=0.3)
    w.weight("net.x_embedder.proj.1.weight", (D, 68))
    w.weight("net.t_embedder.1.linear_1.weight", (D, D))
    w.weight("net.t_embedder.1.linear_2.weight", (3 * D, D), gain=0.3)
    w.norm("net.t_embedding_norm.weight", (D,))
    w.weight("net.final_layer.adaln_modulation.1.weight", (256, D))
    w.weight("net.final_layer.adaln_modulation.2.weight", (2 * D, 256), gain=0.3)
    w.weight("net.final_layer.linear.weight", (64, D))
    for i in range(6):
        p = "net.llm_adapter.blocks.%d." % i
        w.norm(p + "norm_self_attn.weight", (AD,))
        w.norm(p + "norm_cross_attn.weight", (AD,))
        w.norm(p + "norm_mlp.weight", (AD,))
        for a in ("self_attn", "cross_attn"):
            for q in ("q_proj", "k_proj", "v_proj", "o_proj"):
                w.weight(p + a + "." + q + ".weight", (AD, AD), gain=0.5 if q == "o_proj" else 1.0)
            w.norm(p + a + ".q_norm.weight", (64,))
            w.norm(p + a + ".k_norm.weight", (64,))
        w.weight(p + "mlp.0.weight", (4 * AD, AD))
        w.bias(p + "mlp.0.bias", 4 * AD)
        w.weight(p + "mlp.2.weight", (AD, 4 * AD), gain=0.5)
        w.bias(p + "mlp.2.bias", AD)
    w.weight("net.llm_adapter.embed.weight", (T5_VOCAB, AD), fan_in=3)      # unit-variance embedding rows
    w.weight("net.llm_adapter.out_proj.weight", (AD, AD))
    w.bias("net.llm_adapter.out_proj.bias", AD)
    w.norm("net.llm_adapter.norm.weight", (AD,))
    return w.save(path)


def write_text_encoder(path, seed=2, layers=2, ff=3072):
    w = _Writer(seed)
    w.weight("model.embed_tokens.weight", (TE_VOCAB, 1024), fan_in=3)
    for i in range(layers):
        p = "model.layers.%d." % i
        w.norm(p + "input_layernorm.weight", (1024,))
        w.norm(p + "post_attention_layernorm.weight", (1024,))
        w.weight(p + "self_attn.q_proj.weight", (2048, 1024))       # 16 heads of 128
        w.weight(p + "self_attn.k_proj.weight", (1024, 1024))       # 8 key/value heads
        w.weight(p + "self_attn.v_proj.weight", (1024, 1024))
        w.weight(p + "self_attn.o_proj.weight", (1024, 2048), gain=0.5)
        w.norm(p + "self_attn.q_norm.weight", (128,))
        w.norm(p + "self_attn.k_norm.weight", (128,))
        w.weight(p + "mlp.gate_proj.weight", (ff, 1024))
        w.weight(p + "mlp.up_proj.weight", (ff, 1024))
        w.weight(p + "mlp.down_proj.weight", (1024, ff), gain=0.5)
    w.norm("model.norm.weight", (1024,))
    return w.save(path)


def write_vae(path, seed=3, dim=96, z=16):
    w = _Writer(seed)

    def res(p, cin, cout):
        w.norm(p + "residual.0.gamma", (cin, 1, 1, 1))
        w.weight(p + "residual.2.weight", (cout, cin, 3, 3, 3), fan_in=cin * 9)     # only the last temporal tap is used
        w.bias(p + "residual.2.bias", cout)
        w.norm(p + "residual.3.gamma", (cout, 1, 1, 1))
        w.weight(p + "residual.6.weight", (cout, cout, 3, 3, 3), gain=0.5, fan_in=cout * 9)
        w.bias(p + "residual.6.bias", cout)
        if cin != cout:
            w.weight(p + "shortcut.weight", (cout, cin, 1, 1, 1))
            w.bias(p + "shortcut.bias", cout)

    def attn(p, c):
        w.norm(p + "norm.gamma", (c, 1, 1))
        w.weight(p + "to_qkv.weight", (3 * c, c, 1, 1))
        w.bias(p + "to_qkv.bias", 3 * c)
        w.weight(p + "proj.weight", (c, c, 1, 1), gain=0.5)
        w.bias(p + "proj.bias", c)

    top = 4 * dim
    # decoder: latent -> conv2 (1x1) -> conv1 -> middle -> four stages of three blocks, 2x upsampling after the first three
    w.weight("conv2.weight", (z, z, 1, 1, 1))
    w.bias("conv2.bias", z)
    w.weight("decoder.conv1.weight", (top, z, 3, 3, 3), fan_in=z * 9)
    w.bias("decoder.conv1.bias", top)
    res("decoder.middle.0.", top, top)
    attn("decoder.middle.1.", top)
    res("decoder.middle.2.", top, top)
    idx, cin = 0, top
    for s, cout in enumerate((top, top, 2 * dim, dim)):
        for _ in range(3):
            res("decoder.upsamples.%d." % idx, cin, cout)
            cin = cout
            idx += 1
        if s < 3:
            w.weight("decoder.upsamples.%d.resample.1.weight" % idx, (cout // 2, cout, 3, 3))
            w.bias("decoder.upsamples.%d.resample.1.bias" % idx, cout // 2)
            cin = cout // 2
            idx += 1
    w.norm("decoder.head.0.gamma", (dim, 1, 1, 1))
    w.weight("decoder.head.2.weight", (3, dim, 3, 3, 3), fan_in=dim * 9)
    w.bias("decoder.head.2.bias", 3)
    # encoder: four stages of two blocks, stride-2 downsampling after the first three
    w.weight("encoder.conv1.weight", (dim, 3, 3, 3, 3), fan_in=27)
    w.bias("encoder.conv1.bias", dim)
    idx, cin = 0, dim
    for s, cout in enumerate((dim, 2 * dim, top, top)):
        for _ in range(2):
            res("encoder.downsamples.%d." % idx, cin, cout)
            cin = cout
            idx += 1
        if s < 3:
            w.weight("encoder.downsamples.%d.resample.1.weight" % idx, (cout, cout, 3, 3))
            w.bias("encoder.downsamples.%d.resample.1.bias" % idx, cout)
            idx += 1
    res("encoder.middle.0.", top, top)
    attn("encoder.middle.1.", top)
    res("encoder.middle.2.", top, top)
    w.norm("encoder.head.0.gamma", (top, 1, 1, 1))
    w.weight("encoder.head.2.weight", (2 * z, top, 3, 3, 3), fan_in=top * 9)
    w.bias("encoder.head.2.bias", 2 * z)
    w.weight("conv1.weight", (2 * z, 2 * z, 1, 1, 1))
    w.bias("conv1.bias", 2 * z)
    return w.save(path)


def write_lora(path, seed=4, rank=16, alpha=8.0, blocks=range(28),
               modules=("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.output_proj",
                        "cross_attn.q_proj", "cross_attn.output_proj", "mlp.layer1", "mlp.layer2")):
    """A LoRA file as the engine's loader pairs it up (engine/src/engine.h:136-170): <module>.lora_down.weight [rank, in],
    <module>.lora_up.weight [out, rank], <module>.alpha (scalar); module names under the "diffusion_model." prefix."""
    shapes = {"self_attn.q_proj": (D, D), "self_attn.k_proj": (D, D), "self_attn.v_proj": (D, D), "self_attn.output_proj": (D, D),
              "cross_attn.q_proj": (D, D), "cross_attn.k_proj": (D, AD), "cross_attn.v_proj": (D, AD), "cross_attn.output_proj": (D, D),
              "mlp.layer1": (FF, D), "mlp.layer2": (D, FF)}
    w = _Writer(seed)
    for i in blocks:
        for m in modules:
            out, inp = shapes[m]
            p = "diffusion_model.blocks.%d.%s" % (i, m)
            w.weight(p + ".lora_down.weight", (rank, inp))
            w.weight(p + ".lora_up.weight", (out, rank))
            w.entries.append((p + ".alpha", [], 2 if w.layout_only else _bf16(np.array([alpha], dtype=np.float32))))
    return w.save(path)


def write_all(directory, seed=0, layout_only=False):
    """All files into `directory`. layout_only: sparse files with the real headers and sizes but zero values (instant; enough
    for a loader to walk them)."""
    _Writer.layout_only = bool(layout_only)
    try:
        return _write_all(directory, seed)
    finally:
        _Writer.layout_only = False


def _write_all(directory, seed):
    os.makedirs(directory, exist_ok=True)
    sizes = {
        "anima-base-v1.0.safetensors": write_dit(os.path.join(directory, "anima-base-v1.0.safetensors"), seed + 1),
        "qwen_3_06b_base.safetensors": write_text_encoder(os.path.join(directory, "qwen_3_06b_base.safetensors"), seed + 2),
        "qwen_image_vae.safetensors": write_vae(os.path.join(directory, "qwen_image_vae.safetensors"), seed + 3),
    }
    os.makedirs(os.path.join(directory, "loras"), exist_ok=True)
    sizes["loras/style_a.safetensors"] = write_lora(os.path.join(directory, "loras", "style_a.safetensors"), seed + 4, rank=16, alpha=8.0)
    sizes["loras/style_b.safetensors"] = write_lora(os.path.join(directory, "loras", "style_b.safetensors"), seed + 5, rank=8, alpha=8.0,
                                                    blocks=range(0, 28, 2), modules=("self_attn.q_proj", "cross_attn.output_proj", "mlp.layer2"))
    return sizes


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    s = int(sys.argv[sys.argv.index("--seed") + 1]) if "--seed" in sys.argv else 0
    for name, n in write_all(sys.argv[1], s).items():
        print("%-32s %7.1f MB" % (name, n / 1e6))
