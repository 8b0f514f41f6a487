"""The POSIX stand-ins for the reference engine's Win32-only files (oracle/posix/), checked on the CPU through the reference's
own headers: the memory-mapped safetensors reader against files written by oracle/synthetic_models.py and by hand (every
dtype, a scalar, a truncated file, a missing tensor, '\\' path separators), the image reader on PPM and BMP, and the three
Win32 calls. Needs the reference's headers to compile the harness (KILN_REFERENCE_TREE or BASELINE.json's reference_path);
skipped where they are absent."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def _reference_src():
    tree = os.environ.get("KILN_REFERENCE_TREE")
    if not tree:
        try:
            tree = json.load(open(os.path.join(ROOT, "BASELINE.json"))).get("reference_path")
        except (OSError, ValueError):
            tree = None
    src = os.path.join(tree, "engine", "src") if tree else None
    return src if src and os.path.isfile(os.path.join(src, "safetensors.h")) else None


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    src = _reference_src()
    if not src:
        pytest.skip("the reference's headers are not on this machine")
    exe = str(tmp_path_factory.mktemp("standins") / "standins_check")
    posix = os.path.join(ROOT, "oracle", "posix")
    cmd = ["g++", "-std=c++17", "-O1", "-I" + posix, "-I" + src, os.path.join(ROOT, "tests", "posix_harness", "standins_check.cpp"),
           os.path.join(posix, "safetensors_posix.cpp"), os.path.join(posix, "image_io_posix.cpp"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return lambda *a: subprocess.run([exe, *a], capture_output=True, text=True, timeout=60).stdout.splitlines()


def _write(path, tensors, pad=0, cut=0):
    header, blob = {}, b""
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    header["__metadata__"] = {"format": "pt"}
    h = json.dumps(header).encode() + b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + (blob[:-cut] if cut else blob))


def test_safetensors_reader_every_dtype(harness, tmp_path):
    f32 = np.array([1.5, -2.25, 3.0e-5, 65504.0, -0.0, 7.0], dtype=np.float32)
    f16 = np.array([1.0, -0.5, 6.1e-5, 5.96e-8, 65504.0], dtype=np.float16)          # normal, subnormal, largest
    bf16 = (np.array([1.0, -3.140625, 1e-20, 2.0 ** 100], dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
    tensors = {"a.f32": ("F32", [2, 3], f32.tobytes()), "b.f16": ("F16", [5], f16.tobytes()), "c.bf16": ("BF16", [2, 2], bf16.tobytes()),
               "d.scalar": ("F32", [], np.float32(8.0).tobytes()), "e.i64": ("I64", [2], np.array([1, 2], dtype=np.int64).tobytes()),
               "f.u8": ("U8", [3], b"abc")}
    p = str(tmp_path / "every.safetensors")
    _write(p, tensors, pad=5)
    out = harness("tensors", p)
    lines = {l.split()[1]: l for l in out if l.startswith("tensor ")}
    assert set(lines) == set(tensors)                                  # __metadata__ is not a tensor
    vals = lambda name: [float(np.float32(v)) for v in lines[name].split("|")[2].replace("..", " ").split()]    # %.9g round-trips fp32
    assert lines["a.f32"].split("|")[0].split()[2:] == ["F32", "2", "3"] and vals("a.f32") == [float(v) for v in f32[:4]] + [7.0]
    assert vals("b.f16") == [float(v) for v in f16[:4]] + [65504.0]
    assert vals("c.bf16") == [float(v) for v in (bf16.astype(np.uint32) << 16).view(np.float32)] + [2.0 ** 100]
    assert lines["d.scalar"].split("|")[0].split()[2:] == ["F32"] and vals("d.scalar") == [8.0, 8.0]      # shape []: one element
    assert lines["e.i64"].split("|")[0].split()[2:] == ["I64", "2"] and lines["e.i64"].endswith("no float view: unsupported dtype")
    assert lines["f.u8"].split("|")[0].split()[2:] == ["Other", "3"] and lines["f.u8"].endswith("no float view: unsupported dtype")


def test_safetensors_reader_errors_and_separators(harness, tmp_path):
    ok = {"w": ("F32", [4], np.arange(4, dtype=np.float32).tobytes())}
    d = tmp_path / "models"
    d.mkdir()
    _write(str(d / "m.safetensors"), ok)
    out = harness("tensors", str(tmp_path) + "\\models\\m.safetensors")            # the engine joins paths with '\\'
    assert out[0].startswith("tensor w F32 4 | bytes 16 | 0 1 2 3 .. 3")
    assert out[1] == "missing: missing tensor no.such.tensor in " + str(tmp_path) + "\\models\\m.safetensors"
    _write(str(tmp_path / "cut.safetensors"), ok, cut=3)
    assert harness("tensors", str(tmp_path / "cut.safetensors")) == ["exception: truncated safetensors (still downloading?): " + str(tmp_path / "cut.safetensors")]
    with open(tmp_path / "short.safetensors", "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    assert harness("tensors", str(tmp_path / "short.safetensors")) == ["exception: bad safetensors header: " + str(tmp_path / "short.safetensors")]
    assert harness("tensors", str(tmp_path / "absent.safetensors")) == ["exception: cannot open " + str(tmp_path / "absent.safetensors")]


def test_safetensors_reader_on_a_synthetic_lora(harness, tmp_path):
    import synthetic_models
    p = str(tmp_path / "lora.safetensors")
    synthetic_models.write_lora(p, seed=9, rank=4, alpha=2.0, blocks=range(2), modules=("self_attn.q_proj", "mlp.layer2"))
    out = [l for l in harness("tensors", p) if l.startswith("tensor ")]
    names = [l.split()[1] for l in out]
    assert len(names) == 2 * 2 * 3 and "diffusion_model.blocks.1.mlp.layer2.lora_up.weight" in names
    row = {l.split()[1]: l for l in out}
    assert row["diffusion_model.blocks.0.mlp.layer2.lora_down.weight"].split("|")[0].split()[2:] == ["BF16", "4", "8192"]
    assert row["diffusion_model.blocks.0.mlp.layer2.lora_up.weight"].split("|")[0].split()[2:] == ["BF16", "2048", "4"]
    assert row["diffusion_model.blocks.0.self_attn.q_proj.alpha"].split("|")[2].split()[0] == "2"
    v = [float(x) for x in row["diffusion_model.blocks.0.self_attn.q_proj.lora_down.weight"].split("|")[2].replace("..", " ").split()]
    assert all(abs(x) <= np.sqrt(3.0 / 2048) * 1.01 for x in v) and any(x != 0 for x in v)


def test_image_reader(harness, tmp_path):
    rng = np.random.default_rng(3)
    img = rng.integers(0, 256, (5, 7, 3), dtype=np.uint8)
    flat = img.reshape(-1).astype(np.uint64)
    want = int((flat * (np.arange(flat.size) % 251 + 1)).sum())
    with open(tmp_path / "a.ppm", "wb") as f:
        f.write(b"P6\n# a comment\n7 5\n255\n" + img.tobytes())
    line = "image 7 5 105 %d first %d %d %d last %d %d %d" % (want, *img[0, 0], *img[-1, -1])
    assert harness("image", str(tmp_path / "a.ppm")) == [line]
    pitch = (7 * 3 + 3) & ~3
    rows = b"".join(img[y, :, ::-1].tobytes() + b"\0" * (pitch - 21) for y in range(4, -1, -1))        # bottom-up BGR rows
    hdr = b"BM" + struct.pack("<IHHI", 54 + len(rows), 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, 7, 5, 1, 24, 0, len(rows), 2835, 2835, 0, 0)
    with open(tmp_path / "a.bmp", "wb") as f:
        f.write(hdr + rows)
    assert harness("image", str(tmp_path / "a.bmp")) == [line]
    top_down = b"".join(img[y, :, ::-1].tobytes() + b"\0" * (pitch - 21) for y in range(5))
    with open(tmp_path / "b.bmp", "wb") as f:
        f.write(b"BM" + struct.pack("<IHHI", 54 + len(rows), 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, 7, -5, 1, 24, 0, len(rows), 2835, 2835, 0, 0) + top_down)
    assert harness("image", str(tmp_path / "b.bmp")) == [line]
    with open(tmp_path / "c.png", "wb") as f:
        f.write(b"\x89PNG\r\n\x1a\n")
    assert harness("image", str(tmp_path / "c.png"))[0].startswith("image error: no decoder")
    assert harness("image", str(tmp_path / "none.ppm")) == ["image error: cannot open " + str(tmp_path / "none.ppm")]
    with open(tmp_path / "t.ppm", "wb") as f:
        f.write(b"P6 7 5 255\n" + img.tobytes()[:50])
    assert harness("image", str(tmp_path / "t.ppm")) == ["image error: truncated PPM"]


def test_win32_calls(harness, tmp_path):
    d = tmp_path / "sub"
    d.mkdir()
    (d / "x.bin").write_bytes(b"1")
    assert harness("files", str(tmp_path) + "\\sub\\x.bin") == ["exists 1", "icmp 0", "deleted 1", "exists 0"]
    assert not (d / "x.bin").exists()


def test_reference_loaders_accept_the_synthetic_model_files(tmp_path):
    """The reference's own Dit::load / TextEncoder::load / Vae::load (engine/src/dit.cu:11-96, te.cu:6-28, vae.cu:38-130) walk
    the files oracle/synthetic_models.py writes - here as sparse layout-only files - with the weight upload stubbed, and
    see the shapes their forward passes expect. Uses the engine objects oracle/build.py left in oracle/_ref/engine_obj."""
    import shutil
    import synthetic_models
    src = _reference_src()
    obj = os.path.join(ROOT, "oracle", "_ref", "engine_obj")
    need = [os.path.join(obj, f) for f in ("kernels.o", "te.o", "dit.o", "vae.o", "sdops.o", "safetensors_posix.o")]
    if not src or not all(os.path.exists(f) for f in need) or not shutil.which("nvcc"):
        pytest.skip("needs the reference's headers and the engine objects of oracle/build.py --ref")
    exe = str(tmp_path / "loader_check")
    o = str(tmp_path / "loader_check.o")
    r = subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "oracle", "posix"),
                        "-I" + src, "-c", os.path.join(ROOT, "tests", "posix_harness", "loader_check.cu"), "-o", o], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run(["nvcc", "-o", exe, o, *need, "-lcublas", "-Xlinker", "--allow-multiple-definition"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    models = str(tmp_path / "models")
    sizes = synthetic_models.write_all(models, layout_only=True)
    assert sizes["anima-base-v1.0.safetensors"] > 4e9 and os.path.getsize(os.path.join(models, "anima-base-v1.0.safetensors")) > 4e9
    r = subprocess.run([exe, models], capture_output=True, text=True, timeout=120)
    out = r.stdout.splitlines()
    assert r.returncode == 0 and not [l for l in out if l.startswith(("FAILED", "bad "))], out[-5:]
    assert "vae top 384 stages 4 4 fp16 1" in out                          # every conv of the real architecture is on its fp16 path
    assert "up 384: 192>384s 384>384 384>384 rs 192x3456" in out and "up 96: 96>96 96>96 96>96 rs 0x0" in out
    assert "down 192: 96>192s 192>192 ds 192x1728" in out and "vae head 3x864 ehead 32x3456 q 32x32" in out
    assert "dit named 685 prefix net. blocks 28 adapter 6" in out
    w = dict(l.split()[1:] for l in out if l.startswith("w "))
    assert w["blocks.0.self_attn.q_proj.weight"] == "2048x2048" and w["blocks.0.cross_attn.k_proj.weight"] == "2048x1024"
    assert w["blocks.0.mlp.layer1.weight"] == "8192x2048" and w["blocks.0.adaln_modulation_mlp.2.weight"] == "6144x256"
    assert w["x_embedder.proj.1.weight"] == "2048x68" and w["final_layer.linear.weight"] == "64x2048" and w["t_embedder.1.linear_2.weight"] == "6144x2048"
    assert w["llm_adapter.blocks.0.mlp.0.weight"] == "4096x1024" and w["llm_adapter.embed.weight"] == "32768x1024"
    assert "te layers 2 ff 3072 vocab 65536 q 2048x1024 k 1024x1024 o 1024x2048" in out
