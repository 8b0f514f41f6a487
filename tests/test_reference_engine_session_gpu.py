"""Protocol-level sessions of the reference's OWN engine, built on Linux twice: over its own kernels and over the library.

The reference's engine (engine/src/main.cpp:620-795) reads one JSON request per line on stdin and writes one JSON event
per line on stdout (docs/GRAPH_PROTOCOL.md; engine/run_job.bat:1-4 is the same pattern as a one-shot run). oracle/build.py
compiles its unchanged sources into oracle/_ref/kiln-engine-ref and, with the five attention-path ops bound to this
repository's library (oracle/ref_ops_binding.h), into oracle/_ref/kiln-engine-shim. Both read the same seeded random model
files (oracle/synthetic_models.py: the real architecture, 28 DiT blocks). The tests drive both with the same scripted
session and check that
  * the event stream is the same, request by request (ready, info, loading, encoded, step i of n, decoded, done),
  * every step preview and the final RGB8 image of the build over the library is as close to the engine's exact-arithmetic
    render (the job's "precision": "fp32") as the reference's own fp16 build is, within a stated factor,
  * the engine's own latent comparison (main.cpp:493-531, --repeat) says the same of the sampled latents.
Nothing under the reference tree is read at run time: the two executables are built beforehand and travel with the tests.
"""
import base64
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
ENGINE_REF = os.path.join(ROOT, "oracle", "_ref", "kiln-engine-ref")
ENGINE_SHIM = os.path.join(ROOT, "oracle", "_ref", "kiln-engine-shim")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (os.path.exists(ENGINE_REF) and os.path.exists(ENGINE_SHIM)),
                                 reason="the reference engine was not built (oracle/build.py --ref DIR)")]

W, H, STEPS = 512, 768, 4          # the reference's default render size (main.cpp:575-576): 1536 image tokens
# the engine takes all free memory for its scratch arena unless it is told to share the card (main.cpp:656-663); the build
# over the library allocates its staging workspace beside the arena, so both builds run with the same budget
ENGINE_ARGS = ["--vram-budget", "30000"]
# how much further from the exact render the build over the library may be than the reference's own fp16 build
FACTOR, FLOOR_LEVELS, FLOOR_REL = 1.5, 0.75, 2e-3


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    import synthetic_models
    d = str(tmp_path_factory.mktemp("kiln_models"))
    synthetic_models.write_all(d, seed=0)
    yield d
    import shutil
    shutil.rmtree(d, ignore_errors=True)


def _cond(rng, n_qwen, n_t5):
    return {"qwen_ids": [int(v) for v in rng.integers(0, 4096, n_qwen)],
            "t5_ids": [int(v) for v in rng.integers(2, 4096, n_t5)],
            "t5_weights": [float(v) for v in np.round(rng.uniform(0.8, 1.2, n_t5), 3)]}


def _job(job_id, out, **extra):
    rng = np.random.default_rng(11)
    j = {"cmd": "generate", "id": job_id, "width": W, "height": H, "steps": STEPS, "seed": 7, "out": out, "preview": True}
    j.update(_cond(rng, 23, 31))
    j["neg"] = _cond(rng, 9, 12)
    j.update(extra)
    return j


def _run(engine, models, lines=None, extra_args=(), timeout=900, engine_args=ENGINE_ARGS):
    env = dict(os.environ, KILN_TC16="1")     # the fp16-activation path on in both builds, not decided by a timing race
    p = subprocess.run([engine, "--models", models, *engine_args, *extra_args],
                       input=("\n".join(json.dumps(l) for l in lines) + "\n").encode() if lines is not None else b"",
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=env, timeout=timeout)
    events = [json.loads(l) for l in p.stdout.decode().splitlines() if l.strip()]
    return p.returncode, events, p.stderr.decode()


def _shape(ev):
    """What of an event must not depend on which kernels ran."""
    keep = {k: ev[k] for k in ("id", "ev", "stage", "step", "of", "what", "w", "h", "out", "skipped_decode", "node", "class_type",
                               "status", "index", "kind", "prefix") if k in ev}
    if ev.get("ev") == "log":
        keep["unknown"] = ev.get("msg", "").startswith("unknown cmd")
    return keep


def _previews(events, job_id):
    out = []
    for e in events:
        if e.get("id") == job_id and e.get("ev") == "step":
            pv = e["preview"]
            out.append(np.frombuffer(base64.b64decode(pv["rgb"]), dtype=np.uint8).reshape(pv["h"], pv["w"], 3).astype(np.float64))
    return out


def _image(path, w=W, h=H):
    img = np.fromfile(path, dtype=np.uint8)
    assert img.size == w * h * 3, "the engine writes raw RGB8 rows (engine.h:560-578)"
    return img.astype(np.float64)


def test_scripted_session_matches_the_reference_engine(models, tmp_path):
    outs = {k: str(tmp_path / (k + ".rgb")) for k in ("ref_nag", "ref_cfg", "ref_exact", "shim_nag", "shim_cfg", "shim_exact")}

    def session(tag):
        return [{"cmd": "info", "id": "i1"},
                _job("nag", outs[tag + "_nag"], nag={"enabled": True, "scale": 5.0, "tau": 2.5, "alpha": 0.25}),   # NAG cross-attention
                {"cmd": "no-such-command", "id": "x"},
                # two contexts per step, then the hires pass: resize to 768 x 1152, VAE encode, two more steps at 3456 image tokens
                _job("cfg", outs[tag + "_cfg"], cfg=3.0, steps=3, hires={"scale": 1.5, "denoise": 0.5, "steps": 2}),
                _job("dropped", outs[tag + "_nag"] + ".never", nag={"enabled": True}),
                {"cmd": "cancel", "id": "not-queued"},
                {"cmd": "cancel", "id": "dropped"},
                _job("exact", outs[tag + "_exact"], nag={"enabled": True}, precision="fp32"),                      # the engine's exact arithmetic
                {"cmd": "info", "id": "i2"}]

    rc_r, ev_r, err_r = _run(ENGINE_REF, models, session("ref"))
    assert rc_r == 0, (ev_r[-3:], err_r[-2000:])
    rc_s, ev_s, err_s = _run(ENGINE_SHIM, models, session("shim"))
    assert rc_s == 0, (ev_s[-3:], err_s[-2000:])
    assert not [e for e in ev_r + ev_s if e.get("ev") in ("error", "fatal")], [e for e in ev_r + ev_s if e.get("ev") in ("error", "fatal")]

    # 1. the protocol: the same events in the same order for every request id, and for the id-less engine events (ready,
    #    loading). The reader thread answers info / unknown / cancel while the worker thread renders (main.cpp:716-790), so
    #    the interleaving BETWEEN ids is not part of the protocol. Log lines carry timings and are not compared, except that
    #    both builds report the unknown command.
    def streams(events):
        by_id = {}
        for e in events:
            if e.get("ev") == "log" and not e.get("msg", "").startswith("unknown cmd"):
                continue
            k = _shape(e)
            if "out" in k:
                k["out"] = os.path.basename(k["out"]).split("_", 1)[1]
            by_id.setdefault(e.get("id"), []).append(k)
        return by_id
    st_r, st_s = streams(ev_r), streams(ev_s)
    assert st_s == st_r
    assert [e["ev"] for e in st_r[None] if e["ev"] != "loading"] == ["ready", "log"] and st_r[None][-1]["unknown"]
    assert [e["ev"] for e in st_r["i1"]] == ["info"] and [e["ev"] for e in st_r["i2"]] == ["info"]
    assert st_r["dropped"] == [{"id": "dropped", "ev": "cancelled"}]          # cancelled while queued: never rendered
    for job, n in (("nag", STEPS), ("cfg", 3), ("exact", STEPS)):
        base = [e for e in st_r[job] if e.get("stage", "base") == "base"]
        assert [e["ev"] for e in base] == ["encoded"] + ["step"] * n + ["decoded", "done"], st_r[job]
        assert [(e["step"], e["of"]) for e in base if e["ev"] == "step"] == [(i + 1, n) for i in range(n)]
        hs = [(e["step"], e["of"]) for e in st_r[job] if e["ev"] == "step" and e.get("stage") == "hires"]
        # the hires pass runs a truncated schedule (denoise 0.5): at least one step, numbered 1..n of n
        assert (len(hs) >= 1 and hs == [(i + 1, len(hs)) for i in range(len(hs))]) if job == "cfg" else hs == [], hs
        scale = 1.5 if job == "cfg" else 1.0
        assert st_r[job][-1]["w"] == int(W * scale) and st_r[job][-1]["h"] == int(H * scale)
    info = [e for e in ev_s if e["ev"] == "info"][0]
    assert info["family"] == "anima" and info["tc"] is True and info["features"]["ext"] is True

    # 2. the renders: both builds' exact jobs agree (the binding leaves the exact path alone) ...
    exact_r, exact_s = _image(outs["ref_exact"]), _image(outs["shim_exact"])
    assert np.abs(exact_r - exact_s).mean() <= 0.05, np.abs(exact_r - exact_s).mean()
    assert exact_r.std() > 8.0, "a flat image would compare nothing"
    # ... and the fp16 NAG job of the build over the library is as close to the exact render as the reference's fp16 build
    err_ref = np.abs(_image(outs["ref_nag"]) - exact_r).mean()
    err_shim = np.abs(_image(outs["shim_nag"]) - exact_r).mean()
    print("image, mean |fp16 - exact| in 8-bit levels: reference %.3f, over the library %.3f" % (err_ref, err_shim))
    assert err_shim <= FACTOR * err_ref + FLOOR_LEVELS
    pv_exact = _previews(ev_r, "exact")
    assert len(_previews(ev_r, "nag")) == len(_previews(ev_s, "nag")) == len(pv_exact) == STEPS
    for i in range(STEPS):
        e_ref = np.abs(_previews(ev_r, "nag")[i] - pv_exact[i]).mean()
        e_shim = np.abs(_previews(ev_s, "nag")[i] - pv_exact[i]).mean()
        assert e_shim <= FACTOR * e_ref + FLOOR_LEVELS, (i, e_ref, e_shim)
    # the CFG job has no exact twin in the session: the two fp16 builds against each other, in the same units
    d_cfg = np.abs(_image(outs["ref_cfg"], 768, 1152) - _image(outs["shim_cfg"], 768, 1152)).mean()
    print("image, CFG job, mean |reference - library| in 8-bit levels: %.3f (NAG job, same measure: %.3f)"
          % (d_cfg, np.abs(_image(outs["ref_nag"]) - _image(outs["shim_nag"])).mean()))
    assert d_cfg <= 2.0 * FACTOR * err_ref + 2 * FLOOR_LEVELS


def test_engine_latent_comparison_tool(models, tmp_path):
    """--repeat FILE (main.cpp:493-531): the engine runs the jobs of a file and logs each latent's relative L2 distance from
    the first job's. First job exact, then the fp16 NAG job, then the exact job again: the distances of the build over the
    library against those of the reference's own build."""
    jobs = tmp_path / "jobs.jsonl"
    base = dict(skip_decode=True, preview=False)
    lines = [_job("exact", "", nag={"enabled": True}, precision="fp32", **base),
             _job("nag16", "", nag={"enabled": True}, **base),
             _job("exact_again", "", nag={"enabled": True}, precision="fp32", **base)]
    jobs.write_text("\n".join(json.dumps(l) for l in lines) + "\n")

    def distances(engine):
        rc, events, err = _run(engine, models, extra_args=["--repeat", str(jobs)])
        assert rc == 0, (events[-3:], err[-2000:])
        msgs = [e["msg"] for e in events if e.get("ev") == "log" and "latent vs job 1" in e.get("msg", "")]
        assert len(msgs) == 2, [e for e in events if e.get("ev") in ("log", "error", "fatal")][-8:]
        assert all("0 pre-existing weights changed" in m for m in msgs)        # the engine's own weight-integrity check
        return [float(m.split("rel_l2")[1]) for m in msgs]

    ref16, ref_again = distances(ENGINE_REF)
    lib16, lib_again = distances(ENGINE_SHIM)
    print("latent rel_l2 against the exact job: reference fp16 %.3e, over the library %.3e" % (ref16, lib16))
    assert ref_again == 0.0 and lib_again == 0.0          # identical jobs give identical latents in both builds
    assert lib16 <= FACTOR * ref16 + FLOOR_REL


def test_graph_request_with_stacked_loras(models, tmp_path):
    """A "graph" request (docs/GRAPH_PROTOCOL.md: a ComfyUI API-format workflow) at 1024 x 1024 = 4096 image tokens: loaders,
    two stacked LoRAs kept unmerged (engine.h:78-170; the binding hands them to the library's second GEMM product), the NAG
    sampler node, decode, save. Three runs: the reference's build, the build over the library, and the reference's build with
    --fp32 (main.cpp:643: every GEMM and attention exact) as the yardstick."""
    GW = GH = 1024
    rng = np.random.default_rng(5)
    graph = {
        "1": {"class_type": "UNETLoader", "inputs": {"unet_name": "anima-base-v1.0.safetensors", "weight_dtype": "default"}},
        "2": {"class_type": "CLIPLoader", "inputs": {"clip_name": "qwen_3_06b_base.safetensors", "type": "stable_diffusion"}},
        "3": {"class_type": "VAELoader", "inputs": {"vae_name": "qwen_image_vae.safetensors"}},
        "4": {"class_type": "LoraLoaderModelOnly", "inputs": {"model": ["1", 0], "lora_name": "style_a.safetensors", "strength_model": 0.8}},
        "5": {"class_type": "LoraLoaderModelOnly", "inputs": {"model": ["4", 0], "lora_name": "style_b.safetensors", "strength_model": -0.5}},
        "6": {"class_type": "ModelSamplingAuraFlow", "inputs": {"model": ["5", 0], "shift": 3.0}},
        "7": {"class_type": "CLIPTextEncode", "inputs": {"clip": ["2", 0], "text": "positive"}},
        "8": {"class_type": "CLIPTextEncode", "inputs": {"clip": ["2", 0], "text": "negative"}},
        "9": {"class_type": "EmptySD3LatentImage", "inputs": {"width": GW, "height": GH, "batch_size": 1}},
        "10": {"class_type": "KSamplerWithNAG", "inputs": {"model": ["6", 0], "positive": ["7", 0], "negative": ["8", 0], "nag_negative": ["8", 0],
                                                          "latent_image": ["9", 0], "seed": 5, "steps": 3, "cfg": 1.0, "sampler_name": "dpmpp_2m",
                                                          "scheduler": "simple", "denoise": 1.0, "nag_scale": 5.0, "nag_tau": 2.5, "nag_alpha": 0.25}},
        "11": {"class_type": "VAEDecode", "inputs": {"samples": ["10", 0], "vae": ["3", 0]}},
        "12": {"class_type": "SaveImage", "inputs": {"images": ["11", 0], "filename_prefix": "session"}},
    }
    tokens = {"7": _cond(rng, 40, 77), "8": _cond(rng, 6, 8)}

    def run(engine, tag, extra=()):
        out_dir = tmp_path / tag
        out_dir.mkdir()
        req = {"cmd": "graph", "id": "g1", "graph": graph, "tokens": tokens, "out_dir": str(out_dir), "preview": True}
        bad = {"cmd": "graph", "id": "g2", "out_dir": str(out_dir),
               "graph": {"1": {"class_type": "NoSuchNode", "inputs": {}}, "2": {"class_type": "SaveImage", "inputs": {"images": ["1", 0]}}}}
        rc, events, err = _run(engine, models, [bad, req], extra_args=extra)
        assert rc == 0, (events[-3:], err[-2000:])
        errors = [e for e in events if e.get("ev") in ("error", "fatal")]
        assert [(e["id"], e.get("node")) for e in errors] == [("g2", "1")], errors        # unsupported node: fails fast, before the GPU
        assert "unsupported node type NoSuchNode" in errors[0]["msg"]
        img_ev = [e for e in events if e.get("ev") == "image"]
        assert len(img_ev) == 1 and img_ev[0]["w"] == GW and img_ev[0]["h"] == GH and img_ev[0]["kind"] == "save" and img_ev[0]["prefix"] == "session"
        lora_log = [e["msg"] for e in events if e.get("ev") == "log" and e.get("msg", "").startswith("LoRA ")]
        assert lora_log and "style_a.safetensors: 224 layers" in lora_log[0] and "style_b.safetensors: 42 layers" in lora_log[0], lora_log
        shapes = []
        for e in events:
            if e.get("id") == "g1":
                k = _shape(e)
                if "out" in k:
                    k["out"] = k["out"].replace("\\", "/").rsplit("/", 1)[1]
                shapes.append(k)
        return shapes, _image(img_ev[0]["out"], GW, GH), _previews(events, "g1")

    sh_r, img_r, pv_r = run(ENGINE_REF, "ref")
    sh_s, img_s, pv_s = run(ENGINE_SHIM, "shim")
    sh_x, img_x, pv_x = run(ENGINE_REF, "exact", extra=["--fp32"])
    assert sh_s == sh_r == sh_x
    assert [e["ev"] for e in sh_r][-1] == "done" and sum(e["ev"] == "step" for e in sh_r) == 3
    started = [e["class_type"] for e in sh_r if e["ev"] == "node" and e.get("status") == "start"]
    assert set(started) >= {"KSamplerWithNAG", "VAEDecode", "SaveImage"}, started
    assert img_x.std() > 8.0
    err_ref, err_lib = np.abs(img_r - img_x).mean(), np.abs(img_s - img_x).mean()
    print("graph at 1024 x 1024 with two LoRAs, image, mean |fp16 - exact| in 8-bit levels: reference %.3f, over the library %.3f" % (err_ref, err_lib))
    assert err_lib <= FACTOR * err_ref + FLOOR_LEVELS
    assert len(pv_r) == len(pv_s) == len(pv_x) == 3
    for a, b, x in zip(pv_r, pv_s, pv_x):
        assert np.abs(b - x).mean() <= FACTOR * np.abs(a - x).mean() + FLOOR_LEVELS


def test_engine_bench_mode(models):
    """--bench WxH (main.cpp:77-152): the engine's own DiT-step benchmark - warm forward passes of all 28 blocks with the
    cross-attention K/V cached, its fp16-activation path against its fp32-input path, a batched CFG step and its per-category
    profile - at the three image sizes of the headline metric (1536 / 3456 / 4096 image tokens), in both builds. Wall-clock
    milliseconds as the engine prints them (whole milliseconds); the build over the library must not be slower."""
    import re
    rows = []
    lora = os.path.join(models, "loras", "style_a.safetensors")      # rank 16 on eight linears of every block, left unmerged
    for size, extra in (("512x768", []), ("768x1152", []), ("1024x1024", []), ("1024x1024", ["--lora", lora])):
        got = {}
        for tag, engine in (("reference", ENGINE_REF), ("library", ENGINE_SHIM)):
            rc, events, err = _run(engine, models, extra_args=["--bench", size, *extra])
            assert rc == 0, (events[-3:], err[-2000:])
            logs = [e["msg"] for e in events if e.get("ev") == "log"]
            assert not [e for e in events if e.get("ev") in ("error", "fatal")]
            step = [m for m in logs if "ms/step (avg of" in m]
            paths = [m for m in logs if m.startswith("fp32-input tensor-core path")]
            cfg = [m for m in logs if m.startswith("CFG step")]
            assert len(step) == 1 and len(paths) == 1 and len(cfg) == 1, logs
            got[tag] = dict(step=float(re.search(r": (\d+) ms/step", step[0]).group(1)),
                            f16=float(re.search(r"fp16-activation path (\d+) ms/step", paths[0]).group(1)),
                            rel=float(re.search(r"rel_l2 ([0-9.e+-]+)", paths[0]).group(1)),
                            cfg=float(re.search(r"batched (\d+) ms", cfg[0]).group(1)))
            if extra:
                assert any(m.startswith("LoRA style_a.safetensors: 224 layers") for m in logs), logs[:12]
            print("--bench %s%s, %s build:" % (size, " with a LoRA" if extra else "", tag))
            for m in logs[logs.index(step[0]):]:
                print("    " + m)
        rows.append((size + (" +LoRA" if extra else ""), got))
    print("size        DiT step ms (reference / library)   batched CFG step ms   fp16 path vs fp32-input path rel_l2")
    for size, g in rows:
        print("%-15s  %5.0f / %-5.0f                       %5.0f / %-5.0f         %.2e / %.2e"
              % (size, g["reference"]["step"], g["library"]["step"], g["reference"]["cfg"], g["library"]["cfg"],
                 g["reference"]["rel"], g["library"]["rel"]))
        assert g["library"]["step"] <= g["reference"]["step"]
        assert g["library"]["cfg"] <= g["reference"]["cfg"]
        assert g["library"]["rel"] <= FACTOR * g["reference"]["rel"] + FLOOR_REL


def test_engine_train_bench_mode(models):
    """--train-bench WxH (main.cpp:330-367): three LoRA training steps (rank 32 on every linear of the 28 blocks; forward,
    backward through every block, the engine's exact attention backward of train.cu:216-242) with its loss and per-category
    profile. In the build over the library the trainer's attention_bwd goes to kb_attn_bwd (oracle/ref_engine_train_bind.cu)
    and its forward attention calls to the library as everywhere else. 512 x 512 (1024 tokens): the largest size whose step
    scratch (train.h:40-42) fits the 800 MB arena the engine keeps when it shares the card; without --vram-budget the arena
    takes all memory and the trainer's own allocations (train.cu:384) fail in the reference's build as well."""
    import re
    got = {}
    for tag, engine in (("reference", ENGINE_REF), ("library", ENGINE_SHIM)):
        rc, events, err = _run(engine, models, extra_args=["--train-bench", "512x512"])
        logs = [e["msg"] for e in events if e.get("ev") == "log"]
        assert rc == 0 and not [e for e in events if e.get("ev") in ("error", "fatal")], (logs[-6:], err[-2000:])
        steps = [re.search(r"step (\d) ([0-9.]+) s, loss ([0-9.eE+-]+)", m) for m in logs if "tokens): step" in m]
        assert len(steps) == 3, logs
        bwd = [m for m in logs if m.strip().startswith("bwd_attention")]
        assert len(bwd) == 1, logs
        got[tag] = dict(sec=[float(s.group(2)) for s in steps], loss=[float(s.group(3)) for s in steps],
                        bwd_ms=float(re.search(r"([0-9.]+) ms", bwd[0]).group(1)))
        print("--train-bench 512x512, %s build:" % tag)
        for m in logs[[i for i, m in enumerate(logs) if "tokens): step" in m][0]:]:
            print("    " + m)
    r, l = got["reference"], got["library"]
    print("train step seconds (reference / library): %s / %s; attention backward in the profiled step: %.1f / %.1f ms; losses %s / %s"
          % (r["sec"], l["sec"], r["bwd_ms"], l["bwd_ms"], r["loss"], l["loss"]))
    assert all(np.isfinite(r["loss"])) and all(np.isfinite(l["loss"]))
    # the first step's loss depends on the forward pass only, the later ones on the updates the gradients produced
    assert abs(l["loss"][0] - r["loss"][0]) <= 2e-3 * abs(r["loss"][0]) + 1e-4
    for a, b in zip(r["loss"][1:], l["loss"][1:]):
        assert abs(a - b) <= 2e-2 * abs(a) + 1e-3, (r["loss"], l["loss"])
    assert l["bwd_ms"] < r["bwd_ms"]
    assert l["sec"][2] <= 1.15 * r["sec"][2] + 0.02          # wall clock of one step, printed to 10 ms: not slower beyond its noise
