"""Benchmark of the serving step: decode tokens per second of a Llama shaped model with random
weights on one B200, with prefill, roofline fractions and an end-to-end figure.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference] [--shape 1b|3b|8b]

Default (`--shape 1b`): a "step" is one decode step of `--batch` requests (256-token prompts, decoding
from position 256 on). W warm-up steps, then regions of exactly K steps each, timed with CUDA events on
the launching stream and synchronised on both sides; `ms_per_step` is the median region. The weights
(2.47 GB) are far larger than L2 (126 MB), so every step streams them from HBM again; no flush is needed.
`e2e` is the whole workload of the reference's own offline benchmark (256-token prompts, 256 outputs,
prefill included) through the Python entry point, host token ids in and out: generated tokens / wall time.

`--impl reference` builds the unmodified arhaamatiq/stride sources kept under baseline/_ref with nvcc and
drives its stock `stride_cli --path tc` on the same model shape and prompts (as its scripts/bench/offline.py
does). `--shape 3b` / `--shape 8b` measure the two larger shapes through the scheduler.
One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import shutil
import statistics
import struct
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _llama(hidden, inter, layers, heads, kv_heads, head_dim, tied, factor, max_pos):
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": hidden, "intermediate_size": inter,
            "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
            "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192},
            "tie_word_embeddings": tied, "rms_norm_eps": 1e-5, "max_position_embeddings": max_pos}


SHAPES = {
    "1b": ("llama-3.2-1b-shape", _llama(2048, 8192, 16, 32, 8, 64, True, 32.0, 4096)),
    "3b": ("llama-3.2-3b-shape", _llama(3072, 8192, 28, 24, 8, 128, True, 32.0, 4096)),
    "8b": ("llama-3.1-8b-shape", _llama(4096, 14336, 32, 32, 8, 128, False, 8.0, 8192)),
}
PROMPT = 256
OUTPUTS = 256
PREFILL_TOKENS = 2048
LONG_CONTEXT = 32768     # cached tokens of the one request of the long-context decode point
REGIONS = 5            # timed regions of K steps each; the median is reported
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


def offline_prompts(count: int, length: int, seed: int = 21) -> list:
    """Token-id prompts made the way arhaamatiq/stride's offline benchmark makes them
    (scripts/bench/offline.py:19-21): the BOS id, then uniform ids, from a seeded generator."""
    rng = random.Random(seed)
    return [[128000] + [rng.randint(1000, 100000) for _ in range(length - 1)] for _ in range(count)]


def describe(name: str, cfg: dict, layers: int, batch: int, page: int, pk: dict) -> dict:
    """The flat `config` record (the same for both arms: it describes the workload, not the program)."""
    return {"model": name, "layers": layers, "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
            "seq_len": cfg["max_position_embeddings"], "prompt_len": PROMPT, "outputs": OUTPUTS, "page_size": page,
            "parallelism": "single-gpu", "l2": "inputs larger than L2: the weights are streamed every step",
            "peaks": pk["source"]}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prefill_flops(cfg: dict, T: int, layers: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2.0 * T * layers * (H * (Hq + 2 * Hkv) * D + Hq * D * H + 3 * H * I)
    attention = layers * 2.0 * 2.0 * Hq * D * (T * (T + 1) / 2.0)
    return linear + attention + 2.0 * H * V


# ---------------------------------------------------------------------------------------------------- the reference arm
REF_DIR = ROOT / "baseline" / "_ref"
REF_SOURCES = ["src/safetensors.cpp", "src/model.cpp", "src/kv_cache.cpp", "src/engine.cpp", "src/scheduler.cpp",
               "src/kernels.cu", "src/device.cu", "src/kernels_tc.cu", "tools/stride_cli.cpp"]


def _json_include() -> str | None:
    """A folder that holds nlohmann/json.hpp (the reference fetches it with CMake; this image carries a copy)."""
    cands = [REF_DIR / "third_party"]
    for p in sys.path:
        cands.append(Path(p) / "include" / "cudnn_frontend" / "thirdparty")
    for c in cands:
        if (c / "nlohmann" / "json.hpp").exists():
            return str(c)
    return None


def build_reference() -> tuple:
    """(path of the reference's stride_cli, how it was built) or (None, why not). The sources are the
    reference's own files, unmodified, copied to baseline/_ref; the flags are those of its CMakeLists.txt:36-44
    with the architecture of this GPU in place of sm_89."""
    cli = REF_DIR / "build" / "stride_cli"
    how = "nvcc -O3 -fmad=false -Xcompiler=-fno-strict-aliasing -DSTRIDE_BACKEND_CUDA, arch sm_100 (CMakeLists.txt:36-44 has 89)"
    if cli.exists():
        return cli, how + "; prebuilt"
    # the unmodified copy under baseline/_ref, else a checkout named by STRIDE_REFERENCE or lying beside this repository
    src = REF_DIR if (REF_DIR / "src").exists() else Path(os.environ.get("STRIDE_REFERENCE", ROOT.parent / "reference"))
    if not (src / "src" / "engine.cpp").exists():
        return None, "the reference's sources are neither under baseline/_ref nor in a checkout beside this repository (STRIDE_REFERENCE)"
    inc = _json_include()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if inc is None or not Path(nvcc).exists():
        return None, "nvcc or nlohmann/json.hpp not found, so the reference cannot be compiled"
    cli.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-fmad=false", "-Xcompiler=-fno-strict-aliasing,-fno-fast-math,-ffp-contract=off,-O3",
           "-gencode", "arch=compute_100,code=[sm_100,compute_100]", "-DSTRIDE_BACKEND_CUDA", f"-I{src / 'src'}", f"-I{inc}",
           *[str(src / s) for s in REF_SOURCES], "-o", str(cli)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0 or not cli.exists():
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-3:]
        return None, "nvcc failed on the reference: " + " | ".join(tail)
    return cli, how


def write_reference_model(folder: Path, cfg: dict, seed: int = 0) -> None:
    """config.json + model.safetensors (bfloat16, N(0, 0.02), norm gains 1 + N(0, 0.1)) for the reference's loader,
    written with torch on the CPU alone: nothing of this repository's engine is imported in the reference arm."""
    import torch
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", True):
        shapes["lm_head.weight"] = (V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (Hq * D, H), p + "self_attn.k_proj.weight": (Hkv * D, H),
                       p + "self_attn.v_proj.weight": (Hkv * D, H), p + "self_attn.o_proj.weight": (H, Hq * D),
                       p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
                       p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,)})
    header, at = {}, 0
    for name in sorted(shapes):
        n = 2
        for s in shapes[name]:
            n *= s
        header[name] = {"dtype": "BF16", "shape": list(shapes[name]), "data_offsets": [at, at + n]}
        at += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    gen = torch.Generator().manual_seed(seed)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in sorted(shapes):
            shape = shapes[name]
            if len(shape) == 1:
                t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
            else:
                t = 0.02 * torch.randn(shape, generator=gen)
            f.write(t.to(torch.bfloat16).view(torch.uint8).numpy().tobytes())


def reference_arm(a) -> int:
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if a.gpus != 1:
        print(f"bench.py: arhaamatiq/stride runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.shape != "1b":
        return unavailable("arhaamatiq/stride takes only a head ratio of 4 and at most 2,048 tokens of context "
                           "(src/model.cpp:49, src/kernels.h:18): the 3B and 8B workloads do not fit it")
    cli, how = build_reference()
    if cli is None:
        return unavailable(how)
    name, cfg = SHAPES["1b"]
    cfg = dict(cfg)
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    pk = peaks()
    tmp = Path(tempfile.mkdtemp(prefix="stride_ref_"))
    try:
        t0 = time.time()
        write_reference_model(tmp / "model", cfg)
        wrote_s = time.time() - t0
        prompts = offline_prompts(64, PROMPT)

        def run(batch: int, max_new: int, path: str = "tc") -> dict:
            """One run of the stock command line, as scripts/bench/offline.py:70-78 calls it."""
            source = tmp / f"p{batch}.jsonl"
            if not source.exists():
                source.write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts[:batch])))
            cmd = [str(cli), "--path", path, "--model", str(tmp / "model"), "--input", str(source), "--output", str(tmp / "o.jsonl"),
                   "--max-new", str(max_new), "--kv-gb", "16", "--concurrency", str(batch), "--max-rows", "2048",
                   "--prefill-chunk", "256", "--max-slots", "256"]
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
            if proc.returncode != 0:
                raise RuntimeError(f"stride_cli exited with {proc.returncode}: " + " | ".join(proc.stderr.strip().splitlines()[-3:]))
            return json.loads(proc.stderr.strip().splitlines()[-1])

        def measure(batch: int, repeats: int, path: str = "tc") -> dict:
            """Generated tokens / run_seconds of the whole run (prefill included), first run discarded; and the
            decode steps alone: the time of the run with 256 outputs less the time of the run with one."""
            whole, first = [], []
            for r in range(repeats + 1):
                d = run(batch, OUTPUTS, path)
                if r > 0:
                    whole.append(d)
            for r in range(repeats):
                first.append(run(batch, 1, path))
            t_whole = statistics.median(d["run_seconds"] for d in whole)
            t_first = statistics.median(d["run_seconds"] for d in first)
            generated = whole[0]["generated"]
            decode_s = max(t_whole - t_first, 1e-9)
            return {"e2e": generated / t_whole, "decode": batch * (OUTPUTS - 1) / decode_s, "ms_per_step": decode_s * 1e3 / (OUTPUTS - 1),
                    "run_seconds": [round(d["run_seconds"], 4) for d in whole], "first_token_seconds": round(t_first, 4),
                    "load_seconds": round(whole[0]["load_seconds"], 2), "steps": whole[0]["steps"], "device": whole[0]["device"]}

        clocks = ClockSampler()
        clocks.start()
        try:
            main = measure(a.batch, 3)
        except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
            clocks.stop()
            return unavailable(f"the reference's stride_cli did not run here: {e}")
        clock_info = clocks.stop()
        points = {}
        if not a.skip_points:
            for b in (1, 64):
                try:
                    m = measure(b, 2)
                    points[f"decode_b{b}"] = round(m["decode"], 1)
                    points[f"e2e_b{b}"] = round(m["e2e"], 1)
                except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
                    points[f"decode_b{b}"] = None
                    points[f"error_b{b}"] = str(e)[:200]
            try:        # its exact (float32) path, the counterpart of this engine's float32 point
                points["decode_b1_float32"] = round(measure(1, 1, "exact")["decode"], 1)
            except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
                points["decode_b1_float32"] = None
                points["error_float32"] = str(e)[:200]
        weight_bytes = 2 * (cfg["num_hidden_layers"] * (cfg["hidden_size"] * (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
                                                      + cfg["num_attention_heads"] * cfg["head_dim"] * cfg["hidden_size"]
                                                      + 3 * cfg["hidden_size"] * cfg["intermediate_size"]) + cfg["vocab_size"] * cfg["hidden_size"])
        kv_token_bytes = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
        step_bytes = weight_bytes + a.batch * (PROMPT + OUTPUTS / 2.0) * kv_token_bytes
        achieved = step_bytes / (main["ms_per_step"] * 1e-3) / 1e9
        print(json.dumps({
            "impl": "reference",
            "metric": f"decode tok/s at batch {a.batch} (Llama 3.2 1B shape, 256-token prompts)", "value": round(main["decode"], 1),
            "unit": "tokens/s", "n_gpus": 1, "steps": OUTPUTS - 1, "warmup": 1, "ms_per_step": round(main["ms_per_step"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids, random weights N(0, 0.02)",
            "config": describe(name, cfg, cfg["num_hidden_layers"], a.batch, 64, pk),
            "clocks": clock_info,
            "e2e": {"value": round(main["e2e"], 1), "unit": "tokens/s",
                    "how": "generated / run_seconds of stride_cli --path tc (256-token prompts, 256 outputs, prefill included), median of 3 after one discarded run"},
            "value_how": "decode steps alone: (run_seconds with 256 outputs - run_seconds with 1 output) / 255 steps; stride_cli prints no device time",
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "points": points,
            "prefill": {"unavailable": "a 2,048-token prompt is refused at intake: the context limit is 2,048 (src/scheduler.cpp:82-89, src/kernels.h:18)"},
            "reference": {"build": how, "device": main["device"], "run_seconds": main["run_seconds"], "first_token_seconds": main["first_token_seconds"],
                          "load_seconds": main["load_seconds"], "engine_steps": main["steps"], "model_written_s": round(wrote_s, 1),
                          "context_capacity": 2048},
        }))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# ---------------------------------------------------------------------------------------------------- this engine
# ---------------------------------------------------------------------------------------------------- another design beside Llama
def _keralorn_config(width: int, ff: int, vocab: int, pairs: int, window: int) -> dict:
    """`pairs` times (windowed attention, lightning), each with a feed-forward, all inside one pass of the loop: the
    attention layer has the heads of the Llama 3.2 1B layer, the lightning layer 16 heads of 128 x 128."""
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": window},
                     "rot": {"dims": 32, "base": 500000.0, "scaling": {"factor": 32.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    heads = width // 128
    lig = {"type": "lightning", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-3 - 5.0 * h / max(heads - 1, 1)) for h in range(heads)]}}
    return {"architecture": "Keralorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [att, lig] * pairs,
            "loop": {"start": 0, "stop": 2 * pairs, "times": 1}}


def _ganupel_config(width: int, ff: int, vocab: int, pairs: int, window: int) -> dict:
    """`pairs` times (recurrent block with a dense PolyNorm feed-forward; sigmoid attention beside HGRN2 with routed experts): the
    attention has the heads of the Llama 3.2 1B layer, HGRN2 16 heads of 128 x 128, the recurrent block `width` channels in
    blocks of 128, and the routed feed-forward eight experts of ff / 4 and one identity expert, two chosen."""
    rec = {"type": "rglru", "mixer": {"width": width, "blocks": width // 128, "conv": 4}, "mlp": {"kind": "dense", "ff": ff}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": window},
                              "rot": {"dims": 64, "base": 500000.0}},
                     "right": {"heads": width // 128, "dim": 128, "vdim": 128}, "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 8, "identity": 1, "top": 2, "scale": 1.0}}}
    return {"architecture": "Ganupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [rec, par] * pairs}


def _pusisun_config(width: int, ff: int, vocab: int, pairs: int, window: int) -> dict:
    """`pairs` times (masked attention, latent attention), each with routed gated experts: the attention has the heads of the Llama
    3.2 1B layer, a window that keeps the first four tokens, slopes and a sink; the latent attention 16 heads of 128 unrotated and 64
    rotated elements over a latent of 512 (a cached row of 576), queries through a latent of 768; eight experts of ff / 4, two chosen."""
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 8, "top": 2}}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": window, "keep_first": 4}}}
    lat = {"type": "latent_attention", "mlp": moe,
           "mixer": {"heads": width // 128, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 768, "kv_rank": 512, "scale": 192 ** -0.5,
                     "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Pusisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [att, lat] * pairs}


def _sitivik_config(width: int, ff: int, vocab: int, pairs: int, window: int) -> dict:
    """Four layers: (windowed attention beside retention), differential attention, (windowed attention beside retention), (chunked
    attention with a sink beside the gated delta rule), each with a gated feed-forward of `ff` and a per-layer token input of 256: the
    windowed and chunked attentions have the heads of the Llama 3.2 1B layer, the differential attention 16 heads of two maps of 64 over
    values of 128, retention and the delta rule 16 heads of 128 x 128 (the delta rule with four taps and low-rank projections of 64)."""
    mlp = {"kind": "dense", "ff": ff}
    left = {"heads": width // 64, "kv_heads": width // 256, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": window}}
    heads = width // 128
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": dict(left, rot={"dims": 64, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}),
                     "right": {"heads": heads, "dim": 128, "vdim": 128, "rot": {"dims": 64, "base": 10000.0},
                               "decay": [1.0 - 2.0 ** (-3 - 5.0 * h / max(heads - 1, 1)) for h in range(heads)]}}}
    dif = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": heads, "kv_heads": max(heads // 4, 1), "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.5, "q_temp": {"coef": 0.1, "every": 256}}}
    par2 = {"type": "parallel_2", "mlp": mlp,
            "mixer": {"left": dict(left, rot={"dims": 32, "base": 500000.0}), "left_scale": 1.0, "right_scale": 1.0,
                      "right": {"heads": heads, "kv_heads": heads, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}}}
    return {"architecture": "Sitivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "token_side": {"dim": 256},
            "layers": ([par, dif] * pairs)[:2 * pairs - 1] + [par2]}


def design_compare(a) -> int:
    """Keralorn at layer sizes of a real model beside LlamaForCausalLM with as many layers of the same width, heads and
    feed-forward (random weights, bfloat16 engine): a prompt of 2,048 tokens in one step, decode steps at batch 8 and 64
    from CUDA graphs; then Keralorn's own kernels alone against their rooflines. One JSON line."""
    import torch
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.kernels import ops

    pk = peaks()
    width, ff, vocab, pairs, page, context = 2048, 8192, 32000, 2, 64, 4096
    layers = 2 * pairs
    llama = _llama(width, ff, layers, width // 64, width // 256, 64, False, 32.0, context)
    llama["vocab_size"] = vocab
    configs = {"keralorn": _keralorn_config(width, ff, vocab, pairs, 1024), "llama": llama}
    if a.design == "ganupel":      # beside the closest design (a recurrence with a state per request and windowed attention) and Llama
        configs = {"ganupel": _ganupel_config(width, ff, vocab, pairs, 1024), **configs}
    if a.design == "pusisun":      # beside the closest design (windowed attention of the same heads, routed experts of the same sizes) and Llama
        configs = {"pusisun": _pusisun_config(width, ff, vocab, pairs, 1024), "ganupel": _ganupel_config(width, ff, vocab, pairs, 1024), "llama": llama}
    if a.design == "sitivik":      # beside the closest design (windowed attention beside a gated linear attention with a state per request) and Llama
        configs = {"sitivik": _sitivik_config(width, ff, vocab, pairs, 1024), "ganupel": _ganupel_config(width, ff, vocab, pairs, 1024), "llama": llama}
    gen = torch.Generator().manual_seed(3)
    out = {"design": a.design, "beside": {"keralorn": "LlamaForCausalLM", "ganupel": "Keralorn, LlamaForCausalLM", "pusisun": "Ganupel, LlamaForCausalLM",
                                          "sitivik": "Ganupel, LlamaForCausalLM"}[a.design], "width": width, "ff": ff, "layers": layers, "vocab": vocab,
           "dtype": "bf16", "data": "synthetic (random weights and tokens)", "peaks": pk,
           "l2": "weights and caches of a step exceed the 126 MB L2; the kernel timings flush L2 between launches"}
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps, prepare=None, clear=False):
        ts = []
        for r in range(reps + 3):
            if prepare:
                prepare()
            if clear:
                flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if r >= 3:
                ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    clocks = ClockSampler()
    clocks.start()
    for name, cfg in configs.items():
        opts = EngineOptions(dtype="bfloat16", max_rows=PREFILL_TOKENS, max_full_rows=64, max_slots=65,
                             kv_pages=64 * 12 + PREFILL_TOKENS // page + 8, page_size=page, max_context=context)
        eng = Engine.from_random(cfg, seed=0, options=opts)
        cache = eng.cache
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        held = {}

        def prefill_prepare():
            if "slot" in held:
                cache.release_slot(held["slot"])
            held["slot"] = cache.acquire_slot()
            cache.ensure(held["slot"], PREFILL_TOKENS)

        ms = timed(lambda: eng.step([StepEntry(held["slot"], 0, toks, [PREFILL_TOKENS - 1])]), 5, prefill_prepare)
        cache.release_slot(held.pop("slot"))
        res = {"prefill_2048_ms": round(ms, 3), "prefill_tok_s": round(PREFILL_TOKENS / ms * 1e3), "weight_bytes_per_step": eng.weight_bytes_per_step(),
               "native_step": eng._program is not None}
        for batch in (8, 64):
            slots = [cache.acquire_slot() for _ in range(batch)]
            prompt = torch.randint(0, vocab, (batch, 512), generator=gen).tolist()
            for b, s_ in enumerate(slots):
                cache.ensure(s_, 512)
                eng.step([StepEntry(s_, 0, prompt[b], [])])
            pos = [512]

            def one():
                entries = []
                for b, s_ in enumerate(slots):
                    cache.ensure(s_, pos[0] + 1)
                    entries.append(StepEntry(s_, pos[0], [prompt[b][pos[0] % 512]], [0]))
                eng.step(entries)
                pos[0] += 1

            for _ in range(a.warmup):
                one()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = min(a.steps, 128)
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            res[f"decode_b{batch}_ms"] = round(ms, 4)
            res[f"decode_b{batch}_tok_s"] = round(batch / ms * 1e3)
            res[f"decode_b{batch}_hbm_fraction_of_measured"] = round(eng.weight_bytes_per_step() / (ms * 1e-3) / (pk["hbm_gbs"] * 1e9), 3)
            for s_ in slots:
                cache.release_slot(s_)
        out[name] = res
        del eng
        torch.cuda.empty_cache()

    if a.design in ("ganupel", "pusisun", "sitivik"):
        out["kernels"] = {"ganupel": _ganupel_kernels, "pusisun": _pusisun_kernels, "sitivik": _sitivik_kernels}[a.design](timed, pk, width, ff)
        out["clocks"] = clocks.stop()
        print(json.dumps(out))
        return 0
    # Keralorn's own kernels alone, beside the like kernel of Llama where there is one
    H, D, V = width // 128, 128, 128
    kern = {}
    dev = "cuda"
    decay = torch.full((H,), 0.99, device=dev)
    for label, entries, length in (("scan_prefill_2048", 1, 2048), ("scan_prefill_8x2048", 8, 2048), ("scan_decode_b64", 64, 1), ("scan_decode_b512", 512, 1)):
        n = entries * length
        proj = torch.randn(1, n, 2 * H * D + 2 * H * V, device=dev)
        state = torch.zeros(entries + 1, H, D, V, device=dev)
        o = torch.empty(n, H * V, device=dev)
        meta = torch.tensor([list(range(entries)), [e * length for e in range(entries)], [length] * entries, [0 if length > 1 else 7] * entries],
                            dtype=torch.int32, device=dev)
        act = torch.empty(n * (2 * H * D + H * V), device=dev)
        ms = timed(lambda: ops.lightning_scan(proj, 0, H * D, 2 * H * D, meta, entries, decay, state, o, H, D, V, act), 5, clear=True)
        flops = 5.0 * n * H * D * V                      # per state element and token: a product, two fused multiply-adds
        moved = 4.0 * (n * (2 * H * D + H * V) + n * H * V + (2 if length == 1 else 1) * entries * H * D * V)
        kern[label] = {"ms": round(ms, 4), "tflops_fp32": round(flops / ms / 1e9, 2), "gb_s": round(moved / ms / 1e6, 1),
                       "hbm_fraction_of_measured": round(moved / (ms * 1e-3) / (pk["hbm_gbs"] * 1e9), 3)}
    for n in (64, 2048):
        proj = torch.randn(1, n, 2 * H * D + 2 * H * V, device=dev)
        o = torch.randn(n, H * V, device=dev)
        y = torch.empty(n, H * V, dtype=torch.bfloat16, device=dev)
        gain = torch.ones(H * V, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.gated_rmsnorm(o, proj, 2 * H * D + H * V, gain, 1e-5, y), 5, clear=True)
        kern[f"gated_rmsnorm_{n}"] = {"ms": round(ms, 4), "gb_s": round(n * H * V * 10.0 / ms / 1e6, 1)}
        h = torch.randn(n, width, device=dev)
        x = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        g, b = torch.ones(width, dtype=torch.bfloat16, device=dev), torch.zeros(width, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.layernorm(h, g, b, 1e-5, x), 5, clear=True)
        ms_r = timed(lambda: ops.rmsnorm(h, g, 1e-5, x), 5, clear=True)
        kern[f"layernorm_{n}"] = {"ms": round(ms, 4), "gb_s": round(n * width * 6.0 / ms / 1e6, 1), "rmsnorm_ms": round(ms_r, 4)}
    out["kernels"] = kern
    out["clocks"] = clocks.stop()
    print(json.dumps(out))
    return 0


def _ganupel_kernels(timed, pk: dict, width: int, ff: int) -> dict:
    """Ganupel's own kernels alone (L2 flushed between launches), each beside the like kernel of Keralorn or Llama."""
    import torch
    from stride_b200.kernels import ops
    dev, kern = "cuda", {}
    hbm = pk["hbm_gbs"] * 1e9

    def record(label, ms, moved=None, flops=None, **more):
        r = {"ms": round(ms, 4)}
        if moved is not None:
            r.update(gb_s=round(moved / ms / 1e6, 1), hbm_fraction_of_measured=round(moved / (ms * 1e-3) / hbm, 3))
        if flops is not None:
            r["tflops"] = round(flops / ms / 1e9, 2)
        r.update(more)
        kern[label] = r

    # the two recurrences, as prompts and as decode steps, beside the decayed recurrence of Keralorn on the same sizes
    H, D, V = width // 128, 128, 128
    for label, entries, length in (("prefill_2048", 1, 2048), ("prefill_8x2048", 8, 2048), ("decode_b64", 64, 1), ("decode_b512", 512, 1)):
        n = entries * length
        meta = torch.tensor([list(range(entries)), [e * length for e in range(entries)], [length] * entries, [0 if length > 1 else 7] * entries],
                            dtype=torch.int32, device=dev)
        act = torch.rand(n, 3 * H * D + H * V, device=dev)
        state = torch.zeros(entries + 1, H, D, V, device=dev)
        o = torch.empty(n, H * V, device=dev)
        ms = timed(lambda: ops.gated_scan(act, 0, H * D, 2 * H * D, 3 * H * D, meta, entries, state, o, H, D, V), 5, clear=True)
        moved = 4.0 * (n * (3 * H * D + H * V) + n * H * V + (2 if length == 1 else 1) * entries * H * D * V)
        record("gated_scan_" + label, ms, moved, 5.0 * n * H * D * V)
        proj = torch.randn(1, n, 2 * H * D + 2 * H * V, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        scratch = torch.empty(n * (2 * H * D + H * V), device=dev)
        ms = timed(lambda: ops.lightning_scan(proj, 0, H * D, 2 * H * D, meta, entries, decay, state, o, H, D, V, scratch), 5, clear=True)
        record("keralorn_scan_" + label, ms, 4.0 * (n * (2 * H * D + H * V) + n * H * V + (2 if length == 1 else 1) * entries * H * D * V),
               5.0 * n * H * D * V)
        C, K = width, 4
        a_, d_, y_ = (torch.rand(n, C, device=dev) for _ in range(3))
        pr = torch.randn(1, n, 2 * C, device=dev)
        xb = torch.zeros(C, device=dev)
        rec = torch.zeros(entries + 1, K, C, device=dev)
        out = torch.empty(n, C, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.rglru_scan(a_, d_, y_, pr, xb, meta, entries, rec, out, K), 5, clear=True)
        record("rglru_scan_" + label, ms, n * C * 14.0 + entries * K * C * 8.0)
    # attention: a prompt of 2,048 tokens and decode steps over 1,024 cached tokens in the window
    Hq, G, Dh, page, window = width // 64, width // 256, 64, 64, 1024
    for label, entries, length, past in (("prefill_2048", 1, 2048, 0), ("decode_b64", 64, 1, 1500)):
        n, per = entries * length, (past + length + page - 1) // page
        pages = torch.randn(entries * per + 1, 2, G, page, Dh, device=dev).to(torch.bfloat16)
        table = torch.arange(entries * per, dtype=torch.int32, device=dev).view(entries, per)
        pos = torch.tensor([past + t for _ in range(entries) for t in range(length)], dtype=torch.int32, device=dev)
        slot = torch.tensor([e for e in range(entries) for _ in range(length)], dtype=torch.int32, device=dev)
        q = torch.randn(n, Hq * Dh, device=dev).to(torch.bfloat16)
        o = torch.empty_like(q)
        bias = torch.zeros(Hq, device=dev)
        meta = torch.tensor([list(range(entries)), [e * length for e in range(entries)], [length] * entries, [past] * entries],
                            dtype=torch.int32, device=dev)
        keys = sum(min(window, past + t + 1) for t in range(length)) * entries
        moved = (2.0 * entries * G * min(window, past + 1) * Dh * 2 + n * Hq * Dh * 4) if length == 1 else None
        ms = timed(lambda: ops.sigmoid_attention_tiles(q, o, pages, table, meta, entries, bias, Hq, G, Dh, Dh, window, 0.125), 5, clear=True)
        record("sigmoid_attention_" + label, ms, flops=4.0 * keys * Hq * Dh, moved=moved,
               fraction_of_measured_bf16=round(6.0 * keys * Hq * Dh / ms / 1e9 / pk["bf16_tflops"], 4))
        ms = timed(lambda: ops.sigmoid_attention(q, o, pages, table, pos, slot, bias, Hq, G, Dh, Dh, window, 0.125), 3, clear=True)
        record("sigmoid_attention_block_per_token_" + label, ms, flops=4.0 * keys * Hq * Dh, moved=moved)
    # the kernels in front of the recurrences and of attention, for a prompt of 2,048 tokens and for 64 decoded tokens
    C, K, B = width, 4, width // 128
    bw = C // B
    gate_w = (torch.randn(B, bw, 2 * bw, device=dev) * 0.05).to(torch.bfloat16)
    vecs = [torch.randn(C, device=dev) * 0.1 for _ in range(5)]
    taps = torch.randn(C, K, device=dev)
    for n in (2048, 64):
        entries = 1 if n == 2048 else n
        pr = torch.randn(1, n, 2 * C, device=dev)
        rec = torch.zeros(entries + 1, K, C, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev) if entries == 1 else torch.full((n,), 9, dtype=torch.int32, device=dev)
        slot = torch.zeros(n, dtype=torch.int32, device=dev) if entries == 1 else torch.arange(n, dtype=torch.int32, device=dev)
        u, a_, d_, y_ = (torch.empty(n, C, device=dev) for _ in range(4))
        ms = timed(lambda: ops.rglru_conv(pr, vecs[0], taps, vecs[1], pos, slot, rec, u), 5, clear=True)
        record(f"rglru_conv_{n}", ms, n * C * 12.0)
        ms = timed(lambda: ops.rglru_gates(gate_w, vecs[2], vecs[3], vecs[4], vecs[0], u, pr, a_, d_, y_), 5, clear=True)
        record(f"rglru_gates_{n}", ms, flops=4.0 * n * C * bw, moved=n * C * 20.0 + gate_w.numel() * 2.0)
        wq = Hq * Dh + 2 * G * Dh
        qkv = torch.randn(1, n, wq, device=dev)
        cs = torch.rand(4096, Dh // 2, 2, device=dev)
        per = (n if entries == 1 else 10 + page - 1) // page + 1
        pages = torch.zeros(entries * per + 1, 2, G, page, Dh, dtype=torch.bfloat16, device=dev)
        table = torch.arange(entries * per, dtype=torch.int32, device=dev).view(entries, per)
        q = torch.empty(n, Hq * Dh, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.qkv_rotate_append(qkv, pos, slot, cs, Dh, q, pages, table, Hq, G, Dh, Dh), 5, clear=True)
        record(f"qkv_rotate_append_{n}", ms, n * wq * 6.0)
        HD = H * D
        proj = torch.randn(1, n, 2 * HD + H * V, device=dev)
        act = torch.empty(n, 3 * HD + H * V, device=dev)
        ms = timed(lambda: ops.hgrn2_activate(proj, vecs[0], vecs[1], act, HD, H * V), 5, clear=True)
        record(f"hgrn2_activate_{n}", ms, n * (5 * HD + 2 * H * V) * 4.0)
    # between the products of the feed-forwards
    for n in (64, 2048):
        up = torch.randn(1, n, ff, device=dev)
        z = torch.empty(n, ff, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.polynorm(up, z, (0.5, 0.3, 0.2, 0.0), 1e-5), 5, clear=True)
        record(f"polynorm_{n}", ms, n * ff * 6.0)
        E, F = 8, ff // 4
        upe = torch.randn(1, n, E * F, device=dev)
        w = torch.zeros(n, E + 1, device=dev)
        w[:, :2] = 0.5
        ze = torch.empty(n, E * F, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.moe_activate(upe, w, ze, E, F), 5, clear=True)
        record(f"moe_activate_{n}", ms, n * E * F * 2.0 + n * 2 * F * 4.0)
        h = torch.randn(n, width, device=dev)
        br = torch.randn(n, width, device=dev)
        parts = torch.randn(2, n, width, device=dev)
        gain = torch.ones(width, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.branch_fold(h, a=br, a_partials=parts, gain=gain), 5, clear=True)
        x = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        ms_r = timed(lambda: ops.rmsnorm(h, gain, 1e-5, x, partials=parts), 5, clear=True)
        record(f"branch_fold_{n}", ms, n * width * 24.0, rmsnorm_with_two_partials_ms=round(ms_r, 4))
    return kern


def _pusisun_kernels(timed, pk: dict, width: int, ff: int) -> dict:
    """Pusisun's own kernels alone (L2 flushed between launches), each beside the like kernel of Ganupel or Llama."""
    import torch
    from stride_b200.kernels import ops
    dev, kern = "cuda", {}
    hbm = pk["hbm_gbs"] * 1e9

    def record(label, ms, moved=None, flops=None, **more):
        r = {"ms": round(ms, 4)}
        if moved is not None:
            r.update(gb_s=round(moved / ms / 1e6, 1), hbm_fraction_of_measured=round(moved / (ms * 1e-3) / hbm, 3))
        if flops is not None:
            r.update(tflops=round(flops / ms / 1e9, 2), fraction_of_measured_bf16=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
        r.update(more)
        kern[label] = r

    def paged(entries, length, past, G, row, planes, page=64):
        n, per = entries * length, (past + length + page - 1) // page
        pages = torch.randn(entries * per + 1, planes, G, page, row, device=dev).to(torch.bfloat16)
        table = torch.arange(entries * per, dtype=torch.int32, device=dev).view(entries, per)
        pos = torch.tensor([past + t for _ in range(entries) for t in range(length)], dtype=torch.int32, device=dev)
        slot = torch.tensor([e for e in range(entries) for _ in range(length)], dtype=torch.int32, device=dev)
        meta = torch.tensor([list(range(entries)), [e * length for e in range(entries)], [length] * entries, [past] * entries],
                            dtype=torch.int32, device=dev)
        return n, pages, table, pos, slot, meta

    # masked attention beside the sigmoid attention of Ganupel: the same heads, window and pages
    Hq, G, Dh, window, keep = width // 64, width // 256, 64, 1024, 4
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / Hq) for h in range(Hq)], device=dev)
    sinks = torch.zeros(Hq, device=dev)
    for label, entries, length, past in (("prefill_2048", 1, 2048, 0), ("decode_b64", 64, 1, 1500)):
        n, pages, table, pos, slot, meta = paged(entries, length, past, G, Dh, 2)
        q = torch.randn(n, Hq * Dh, device=dev).to(torch.bfloat16)
        o = torch.empty_like(q)
        seen = lambda i: min(window, i + 1) + min(keep, max(i + 1 - window, 0))
        keys = sum(seen(past + t) for t in range(length)) * entries
        moved = (2.0 * entries * G * seen(past) * Dh * 2 + n * Hq * Dh * 4) if length == 1 else None
        ms = timed(lambda: ops.masked_attention_tiles(q, o, pages, table, meta, entries, slopes, sinks, Hq, G, Dh, Dh, window, keep, 0.125), 5, clear=True)
        record("masked_attention_" + label, ms, moved, 4.0 * keys * Hq * Dh)
        ms = timed(lambda: ops.sigmoid_attention_tiles(q, o, pages, table, meta, entries, sinks, Hq, G, Dh, Dh, window, 0.125), 5, clear=True)
        keys_s = sum(min(window, past + t + 1) for t in range(length)) * entries
        record("ganupel_sigmoid_attention_" + label, ms, moved, 6.0 * keys_s * Hq * Dh)       # its weights go through the tensor cores as two parts
        ms = timed(lambda: ops.masked_attention(q, o, pages, table, pos, slot, slopes, sinks, Hq, G, Dh, Dh, window, keep, 0.125), 3, clear=True)
        record("masked_attention_block_per_token_" + label, ms, moved, 4.0 * keys * Hq * Dh)
    # latent attention: every earlier key, one cached row of 576 per token read by all 16 heads, the values its first 512 elements
    H, D, R, V, C, Q = width // 128, 128, 64, 128, 512, 768
    row = C + R
    cs = torch.rand(4096, R // 2, 2, device=dev)
    for label, entries, length, past in (("prefill_2048", 1, 2048, 0), ("decode_b64", 64, 1, 1500)):
        n, pages, table, pos, slot, meta = paged(entries, length, past, 1, row, 1)
        ql = torch.randn(n, H * row, device=dev).to(torch.bfloat16)
        ol = torch.empty(n, H * C, dtype=torch.bfloat16, device=dev)
        keys = sum(past + t + 1 for t in range(length)) * entries
        moved = (entries * (past + 1) * row * 2.0 + n * H * (row + C) * 2.0) if length == 1 else None
        ms = timed(lambda: ops.masked_attention_tiles(ql, ol, pages, table, meta, entries, None, None, H, 1, row, C, 0, 0, 0.07), 5, clear=True)
        record("latent_attention_" + label, ms, moved, 2.0 * keys * H * (row + C))
    # the kernels in front of and behind the attentions, for a prompt of 2,048 tokens and for 64 decoded tokens
    for n in (2048, 64):
        entries = 1 if n == 2048 else n
        length, past = (n, 0) if entries == 1 else (1, 9)
        _, pages, table, pos, slot, meta = paged(entries, length, past, G, Dh, 2)
        wq = Hq * Dh + 2 * G * Dh
        qkv = torch.randn(1, n, wq, device=dev)
        bias, qg, kg = torch.randn(wq, device=dev), torch.ones(Hq * Dh, device=dev), torch.ones(G * Dh, device=dev)
        q = torch.empty(n, Hq * Dh, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.qkv_norm_append(qkv, bias, qg, kg, 1e-6, pos, slot, q, pages, table, Hq, G, Dh, Dh), 5, clear=True)
        record(f"qkv_norm_append_{n}", ms, n * wq * 6.0)
        csr = torch.rand(4096, Dh // 2, 2, device=dev)
        ms = timed(lambda: ops.qkv_rotate_append(qkv, pos, slot, csr, Dh, q, pages, table, Hq, G, Dh, Dh), 5, clear=True)
        record(f"ganupel_qkv_rotate_append_{n}", ms, n * wq * 6.0)
        _, lpages, ltable, pos, slot, meta = paged(entries, length, past, 1, row, 1)
        proj = torch.randn(1, n, Q + row, device=dev)
        cq = torch.empty(n, Q, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.latent_prepare(proj, torch.ones(Q, device=dev), torch.ones(C, device=dev), 1e-6, pos, slot, cs, cq, lpages, ltable, Q, C, R),
                   5, clear=True)
        record(f"latent_prepare_{n}", ms, n * (Q + row) * 6.0)
        qp = torch.randn(1, n, H * (D + R), device=dev)
        qh = torch.empty(n, H, D + R, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.rotate_heads(qp, pos, cs, qh.view(n, H * (D + R)), H, D + R, D, R), 5, clear=True)
        record(f"rotate_heads_{n}", ms, n * H * (D + R) * 6.0)
        uk = (torch.randn(H, D, C, device=dev) * 0.05).to(torch.bfloat16)
        uv = (torch.randn(H, C, V, device=dev) * 0.05).to(torch.bfloat16)
        ql = torch.empty(n, H, row, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.head_linear(qh, uk, ql, tail=R), 5, clear=True)
        record(f"head_linear_keys_into_queries_{n}", ms, n * H * (D + R + row) * 2.0 + uk.numel() * 2.0, 2.0 * n * H * D * C)
        ol = torch.randn(n, H, C, device=dev).to(torch.bfloat16)
        mixed = torch.empty(n, H, V, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.head_linear(ol, uv, mixed), 5, clear=True)
        record(f"head_linear_values_{n}", ms, n * H * (C + V) * 2.0 + uv.numel() * 2.0, 2.0 * n * H * C * V)
    # between the products of the feed-forward, and the norm behind a sublayer beside the plain fold and the norm in front
    for n in (64, 2048):
        E, F = 8, ff // 4
        logits = torch.randn(n, E, device=dev)
        w = torch.empty(n, E, device=dev)
        rb = torch.zeros(E, device=dev)
        ms = timed(lambda: ops.moe_route(logits, rb, w, 2, 1.0, biased=True), 5, clear=True)
        record(f"moe_route_{n}", ms, n * E * 8.0)
        upe = torch.randn(1, n, 2 * E * F, device=dev)
        ze = torch.empty(n, E * F, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.moe_activate(upe, w, ze, E, F, gated=True), 5, clear=True)
        record(f"moe_activate_gated_{n}", ms, n * E * F * 2.0 + n * 2 * 2 * F * 4.0)
        up1 = torch.randn(1, n, E * F, device=dev)
        ms = timed(lambda: ops.moe_activate(up1, w, ze, E, F), 5, clear=True)
        record(f"ganupel_moe_activate_{n}", ms, n * E * F * 2.0 + n * 2 * F * 4.0)
        h = torch.randn(n, width, device=dev)
        br = torch.randn(n, width, device=dev)
        parts = torch.randn(2, n, width, device=dev)
        gain = torch.ones(width, dtype=torch.bfloat16, device=dev)
        ms = timed(lambda: ops.branch_norm_fold(h, gain, 1e-6, a=br, a_partials=parts), 5, clear=True)
        ms_f = timed(lambda: ops.branch_fold(h, a=br, a_partials=parts, gain=gain), 5, clear=True)
        x = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        ms_r = timed(lambda: ops.rmsnorm(h, gain, 1e-6, x, partials=parts), 5, clear=True)
        record(f"branch_norm_fold_{n}", ms, n * width * 24.0, ganupel_branch_fold_ms=round(ms_f, 4), rmsnorm_with_two_partials_ms=round(ms_r, 4))
        e = torch.randn(n, width, device=dev)
        ms = timed(lambda: ops.stream_add(h, e, gain, partials=parts), 5, clear=True)
        record(f"stream_add_{n}", ms, n * width * 20.0)
    return kern


def _sitivik_kernels(timed, pk: dict, width: int, ff: int) -> dict:
    """Sitivik's own kernels alone (L2 flushed between launches), each beside the like kernel of Ganupel, Keralorn or Llama."""
    import torch
    from stride_b200.kernels import ops
    from stride_b200.kernels.native import ImmediateProgram
    from stride_b200.parts import Workspace
    from stride_b200.parts.context import step_context
    dev, kern, f32, bf = "cuda", {}, torch.float32, torch.bfloat16
    hbm = pk["hbm_gbs"] * 1e9

    def record(label, ms, moved=None, flops=None, **more):
        r = {"ms": round(ms, 4)}
        if moved is not None:
            r.update(gb_s=round(moved / ms / 1e6, 1), hbm_fraction_of_measured=round(moved / (ms * 1e-3) / hbm, 3))
        if flops is not None:
            r.update(tflops=round(flops / ms / 1e9, 2), fraction_of_measured_bf16=round(flops / ms / 1e9 / pk["bf16_tflops"], 4))
        r.update(more)
        kern[label] = r

    ws = Workspace(dev, 2048)

    def op(ctx, library, function, ints, floats=()):
        """One operation of the step program, launched for the step `ctx` describes."""
        return ImmediateProgram(ctx, None).prepared(library, function, ints, floats)

    Hq, G, Dh, window, page = width // 64, width // 256, 64, 1024, 64
    H, D, V = width // 128, 128, 128
    cs = torch.rand(4096, 32, 2, device=dev)
    for label, entries, length, past in (("prefill_2048", 1, 2048, 0), ("decode_b64", 64, 1, 1500)):
        n, per = entries * length, (past + length + page - 1) // page
        ctx = step_context([(e, length, past) for e in range(entries)], ws, bf, rows=2048)
        pages = torch.randn(entries * per + 1, 2, G, page, Dh, device=dev).to(bf)
        table = torch.arange(entries * per, dtype=torch.int32, device=dev).view(entries, per)
        where = [per, page, pages.stride(0), pages.stride(1), pages.stride(2)]
        q = torch.randn(n, Hq * Dh, device=dev).to(bf)
        o32 = torch.empty(n, Hq * Dh, dtype=f32, device=dev)
        sinks = torch.zeros(Hq, device=dev)
        # windowed and chunked attention (the tile kernel of the masked attention with another mask), beside Ganupel's sigmoid attention
        for name, win, chunk, sink in (("windowed", window, 0, None), ("chunked_sink", 0, window, sinks)):
            lo = (lambda i: max(0, i - window + 1)) if win else (lambda i: i // window * window)
            keys = sum(past + t + 1 - lo(past + t) for t in range(length)) * entries
            moved = (2.0 * entries * G * (past + 1 - lo(past)) * Dh * 2 + n * Hq * Dh * 6) if length == 1 else None
            ms = timed(op(ctx, "masked_attention", "sb_op_masked_attention_tiles",
                          [q, o32, pages, table, *where, None, sink, Hq, G, Dh, Dh, Dh, win, 0, chunk, 1], [0.125]), 5, clear=True)
            record(f"{name}_attention_{label}", ms, moved, 6.0 * keys * Hq * Dh)          # the weights go through the tensor cores as two parts
        obf = torch.empty(n, Hq * Dh, dtype=bf, device=dev)
        meta = ctx.entry_meta
        ms = timed(lambda: ops.sigmoid_attention_tiles(q, obf, pages, table, meta, entries, sinks, Hq, G, Dh, Dh, window, 0.125), 5, clear=True)
        keys_s = sum(min(window, past + t + 1) for t in range(length)) * entries
        record("ganupel_sigmoid_attention_" + label, ms, None, 6.0 * keys_s * Hq * Dh)
        # differential attention: 2 x 16 query heads over 2 x 4 key heads of 64, values of 128 stored once per map, every earlier key
        Hd, Gd = 2 * H, 2 * max(H // 4, 1)
        dpages = torch.randn(entries * per + 1, 2, Gd, page, V, device=dev).to(bf)
        dwhere = [per, page, dpages.stride(0), dpages.stride(1), dpages.stride(2)]
        qd = torch.randn(n, Hd * Dh, device=dev).to(bf)
        od = torch.empty(n, Hd * V, dtype=f32, device=dev)
        keys = sum(past + t + 1 for t in range(length)) * entries
        moved = (entries * Gd * (past + 1) * (Dh + V) * 2.0 + n * Hd * (Dh * 2 + V * 4)) if length == 1 else None
        ms = timed(op(ctx, "masked_attention", "sb_op_masked_attention_tiles", [qd, od, dpages, table, *dwhere, None, None, Hd, Gd, Dh, V, V, 0, 0, 0, 1],
                      [0.125]), 5, clear=True)
        record("differential_attention_" + label, ms, moved, 2.0 * keys * Hd * (Dh + 2 * V))
        # what stands in front of and behind the attentions
        wq = Hq * Dh + 2 * G * Dh
        proj = torch.randn(n * (wq + Hq * Dh), device=dev)
        gains = torch.ones(Hq * Dh, device=dev)
        qo = torch.empty(n, Hq * Dh, dtype=bf, device=dev)
        ms = timed(op(ctx, "masked_attention", "sb_op_qkv_prepare", [proj, wq + Hq * Dh, 1, 0, gains[:wq], gains, gains, 1, cs, 64, 1, 0, qo, bf, pages, table,
                                                                    *where, Hq, G, Dh, Dh, Dh, 1], [1e-6, 0.0]), 5, clear=True)
        record(f"qkv_prepare_norm_rotate_append_{label}", ms, n * wq * 6.0)
        csr = torch.rand(4096, Dh // 2, 2, device=dev)
        qkv = proj[:n * wq].view(1, n, wq)
        ms = timed(lambda: ops.qkv_rotate_append(qkv, ctx.positions, ctx.slots, csr, Dh, qo, pages, table, Hq, G, Dh, Dh), 5, clear=True)
        record(f"ganupel_qkv_rotate_append_{label}", ms, n * wq * 6.0)
        y = torch.empty(n, Hq * Dh, dtype=bf, device=dev)
        ms = timed(op(ctx, "masked_attention", "sb_op_head_gate", [o32, proj, wq + Hq * Dh, 1, 0, wq, y, bf, Hq, G, Dh, 1, 0], [0.0, 1.0, 1e-6]), 5, clear=True)
        record(f"head_gate_elementwise_{label}", ms, n * Hq * Dh * 10.0)
        yd = torch.empty(n, H * V, dtype=bf, device=dev)
        ms = timed(op(ctx, "masked_attention", "sb_op_head_gate", [od, proj, wq + Hq * Dh, 1, 0, wq, yd, bf, H, Gd // 2, V, 2, 1], [0.7, 0.5, 1e-6]), 5, clear=True)
        record(f"head_gate_differential_{label}", ms, n * H * V * 10.0)
        # retention: rotation, the decayed recurrence (Keralorn's kernel, fed ready-made), norm and gate per head
        wr = 2 * H * D + 2 * H * V
        rproj = torch.randn(n * wr, device=dev)
        ready = torch.empty(n * (2 * H * D + H * V), device=dev)
        ms = timed(op(ctx, "lightning", "sb_op_rotate_qk", [rproj, wr, 1, 0, 0, H * D, 2 * H * D, cs, 64, 0, ready, H, D, V], [D ** -0.5]), 5, clear=True)
        record(f"retention_rotate_{label}", ms, n * (2 * H * D + H * V) * 8.0)
        state = torch.zeros(entries + 1, H, D, V, device=dev)
        decay = torch.full((H,), 0.98, device=dev)
        ro = torch.empty(n, H * V, device=dev)
        ms = timed(op(ctx, "lightning", "sb_op_lightning_scan", [ready, 2 * H * D + H * V, 1, 0, 0, H * D, 2 * H * D, decay, state, ro, H, D, V, None, 1]), 5,
                   clear=True)
        record(f"retention_recurrence_{label}", ms, (2.0 * entries * H * D * V * 4) if length == 1 else None, 4.0 * n * H * D * V,
               note="float32 arithmetic: the fraction is of the tensor-core peak only for scale")
        ry = torch.empty(n, H * V, dtype=bf, device=dev)
        ms = timed(op(ctx, "lightning", "sb_op_group_norm_gate", [ro, rproj, wr, 1, 0, 2 * H * D + H * V, None, 0, ry, bf, H, V, 1], [1e-6]), 5, clear=True)
        record(f"group_norm_gate_{label}", ms, n * H * V * 10.0)
        # the gated delta rule: convolution, unit vectors, decays; the recurrence
        C, ra = 2 * H * D + H * V, 64
        w1, w2 = C + H + 2 * ra, H * D + H * V
        p1, p2 = torch.randn(n * w1, device=dev) * 0.5, torch.randn(n * w2, device=dev) * 0.5
        conv = torch.randn(C, 4, device=dev) * 0.3
        record_elems = H * D * V + 3 * C
        rec = torch.zeros(entries + 1, record_elems, device=dev)
        dready = torch.empty(n * (C + H + H * D), device=dev)
        alog, dtb = torch.zeros(H, device=dev), torch.full((H * D,), -4.0, device=dev)
        ms = timed(op(ctx, "delta_rule", "sb_op_delta_prepare", [p1, w1, 1, p2, w2, 1, 0, conv, alog, dtb, rec, record_elems, H * D * V, dready, H, H, D, V, 4]),
                   5, clear=True)
        record(f"delta_prepare_{label}", ms, n * (C * 8.0 + H * D * 8.0))
        do = torch.empty(n, H * V, device=dev)
        ms = timed(op(ctx, "delta_rule", "sb_op_delta_scan", [dready, rec, record_elems, do, H, H, D, V]), 5, clear=True)
        record(f"delta_recurrence_{label}", ms, (2.0 * entries * H * D * V * 4) if length == 1 else None, 8.0 * n * H * D * V,
               note="float32 arithmetic: the fraction is of the tensor-core peak only for scale")
        gproj = torch.rand(n, 3 * H * D + H * V, device=dev)
        go = torch.empty(n, H * V, device=dev)
        gstate = torch.zeros(entries + 1, H, D, V, device=dev)
        try:
            ms = timed(lambda: ops.gated_scan(gproj, 0, H * D, 2 * H * D, 3 * H * D, meta, entries, gstate, go, H, D, V), 5, clear=True)
            record(f"ganupel_gated_recurrence_{label}", ms, (2.0 * entries * H * D * V * 4) if length == 1 else None, 6.0 * n * H * D * V)
        except (AttributeError, TypeError, RuntimeError) as e:
            kern[f"ganupel_gated_recurrence_{label}"] = {"unavailable": str(e)[:120]}
        # the folds: two branches normed one by one; the per-layer token input's cast and gate
        h = torch.randn(n, width, device=dev)
        a_, b_ = torch.randn(n, width, device=dev), torch.randn(n, width, device=dev)
        parts = torch.randn(2 * n * width, device=dev)
        gain = torch.ones(width, device=dev)
        ms = timed(op(ctx, "branch", "sb_op_branch_pair_norm_fold", [h, a_, parts, 1, 0, b_, parts[n * width:], 1, gain, gain, f32, width], [0.5, 0.5, 1e-6]),
                   5, clear=True)
        record(f"branch_pair_norm_fold_{label}", ms, n * width * 32.0)
        gb = torch.ones(width, dtype=bf, device=dev)
        ms = timed(lambda: ops.branch_norm_fold(h, gb, 1e-6, a=a_, a_partials=parts[:2 * n * width].view(2, n, width)), 5, clear=True)
        record(f"pusisun_branch_norm_fold_{label}", ms, n * width * 24.0)
        x = torch.empty(n, width, dtype=bf, device=dev)
        ms = timed(op(ctx, "elementwise", "sb_op_stream_cast", [h, parts, 1, 0, x, bf, width]), 5, clear=True)
        record(f"stream_cast_{label}", ms, n * width * 14.0)
        table_s = torch.randn(32000, 4 * 256, device=dev).to(bf)
        gsum, gout = torch.randn(n * 256, device=dev), torch.empty(n, 256, dtype=bf, device=dev)
        ms = timed(op(ctx, "elementwise", "sb_op_token_gate", [gsum, 256, 1, 0, table_s, bf, 1024, 256, 32000, None, gout, bf, 1]), 5, clear=True)
        record(f"token_gate_{label}", ms, n * 256 * 8.0)
    return kern


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="1b: the decode step (default); 3b, 8b: serving runs")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64, float32 and prefill measurements")
    ap.add_argument("--design", default="", choices=["", "keralorn", "ganupel", "pusisun", "sitivik"],
                    help="keralorn: prefill and decode of that design beside a Llama of equal layer sizes, and its own kernels alone; "
                         "ganupel: the same beside Keralorn and Llama; pusisun: the same beside Ganupel and Llama")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.design:
        return design_compare(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.shape != "1b":
        return serving_shape(a)

    import torch
    from stride_b200 import LLM, Engine, EngineOptions, StepEntry
    from stride_b200.kernels import ops

    name, cfg = SHAPES["1b"]
    cfg = dict(cfg)
    context = cfg["max_position_embeddings"]
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    max_batch = max(a.batch, 1 if a.skip_points else 64)
    page = 64
    regions = max(1, min(REGIONS, (context - PROMPT - a.warmup - 2) // max(a.steps, 1)))
    main_tokens = PROMPT + a.warmup + regions * a.steps + 1
    pages = max(a.batch * -(-main_tokens // page), max_batch * -(-(PROMPT + OUTPUTS + 8) // page)) + PREFILL_TOKENS // page + 8
    opts = EngineOptions(dtype="bfloat16", max_rows=max(PREFILL_TOKENS, max_batch), max_full_rows=max_batch, max_slots=max_batch + 1,
                         kv_pages=pages, page_size=page, max_context=context)
    engine = Engine.from_random(cfg, seed=0, options=opts)
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    kv_token_bytes = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    weight_bytes = engine.weight_bytes_per_step()

    def decode_run(eng, batch: int, steps: int, warmup: int, regions: int):
        """Prefill `batch` prompts of PROMPT tokens, run `warmup` decode steps, then time `regions` regions of exactly
        `steps` decode steps each. Returns ([(ms per step, mean context) per region], launches per step)."""
        cache = eng.cache
        slots = [cache.acquire_slot() for _ in range(batch)]
        prompts = torch.randint(0, vocab, (batch, PROMPT), generator=gen).tolist()
        per_step = max(1, eng.options.max_rows // PROMPT)
        for i in range(0, batch, per_step):
            entries = []
            for s, p in zip(slots[i:i + per_step], prompts[i:i + per_step]):
                cache.ensure(s, PROMPT)
                entries.append(StepEntry(s, 0, p, []))
            eng.step(entries)
        total = warmup + regions * steps
        tokens = torch.randint(0, vocab, (total, batch), generator=gen).tolist()
        out_tok = torch.zeros(batch, dtype=torch.int32, device=eng.device)
        out_val = torch.zeros(batch, dtype=torch.float32, device=eng.device)

        def one(k):
            pos = PROMPT + k
            entries = []
            for b, s in enumerate(slots):
                cache.ensure(s, pos + 1)
                entries.append(StepEntry(s, pos, [tokens[k][b]], [0]))
            logits = eng.step(entries)
            ops.argmax(logits, out_tok, out_val)

        for k in range(warmup):
            one(k)
        out, launches = [], 0
        for r in range(regions):
            torch.cuda.synchronize()
            l0 = ops.launches
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for k in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(k)
            stop.record()
            torch.cuda.synchronize()
            out.append((start.elapsed_time(stop) / steps, PROMPT + warmup + r * steps + (steps + 1) / 2.0))
            launches = (ops.launches - l0) // steps
        for s in slots:
            cache.release_slot(s)
        return out, launches

    def median_region(rs):
        return sorted(rs)[len(rs) // 2]

    def e2e_run(batch: int, repeats: int = 3):
        """The reference's offline workload through the Python entry point: `batch` prompts of 256 host token ids in,
        256 generated ids each back on the host, prefill included; generated / wall seconds, first run discarded."""
        llm = LLM(engine=engine, concurrency=batch, max_rows=opts.max_rows, prefill_chunk=PROMPT)
        prompts = offline_prompts(batch, PROMPT)
        rates = []
        for r in range(repeats + 1):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = llm.generate(prompts, max_new_tokens=OUTPUTS)
            dt = time.perf_counter() - t0
            if r > 0:
                rates.append(sum(len(o.tokens) for o in outs) / dt)
        return statistics.median(rates), llm.last_stats

    def prefill_run(reps: int = 5):
        cache = engine.cache
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        times = []
        for r in range(reps + 1):
            slot = cache.acquire_slot()
            cache.ensure(slot, PREFILL_TOKENS)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry(slot, 0, toks, [PREFILL_TOKENS - 1])])
            stop.record()
            torch.cuda.synchronize()
            if r > 0:
                times.append(start.elapsed_time(stop))
            cache.release_slot(slot)
        return statistics.median(times)

    def long_context_run(ctx: int, steps: int = 16, portion: int = 2048):
        """Milliseconds a decode step of one request that holds `ctx` cached tokens (its prompt fed in portions first)."""
        o = EngineOptions(dtype="bfloat16", max_rows=portion, max_full_rows=1, max_slots=2, kv_pages=ctx // page + 8, page_size=page,
                          max_context=ctx + 256)
        eng = Engine.from_random(cfg, seed=0, options=o)
        cache = eng.cache
        slot = cache.acquire_slot()
        toks = torch.randint(0, vocab, (ctx + steps + 8,), generator=gen).tolist()
        for a0 in range(0, ctx, portion):
            cache.ensure(slot, a0 + portion)
            eng.step([StepEntry(slot, a0, toks[a0:a0 + portion], [])])

        def one(k):
            cache.ensure(slot, ctx + k + 1)
            eng.step([StepEntry(slot, ctx + k, [toks[ctx + k]], [0])])
        for k in range(4):
            one(k)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(4, 4 + steps):
            one(k)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    clocks = ClockSampler()
    clocks.start()
    rs, launches = decode_run(engine, a.batch, a.steps, a.warmup, regions)
    clock_info = clocks.stop()
    ms, mean_ctx = median_region(rs)
    value = a.batch * 1000.0 / ms
    step_bytes = weight_bytes + a.batch * mean_ctx * kv_token_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e, stats = e2e_run(a.batch)
    points, prefill = {}, None
    if not a.skip_points:
        # decoding over the whole 256 outputs of the workload (contexts 256 -> 511), batch 1, 8 and 64
        for b in sorted({1, a.batch, 64}):
            pr, _ = decode_run(engine, b, OUTPUTS - 4, 3, 1)      # positions 256..510: the steps that make outputs 2..256
            points[f"decode_b{b}"] = round(b * 1000.0 / pr[0][0], 1)
        pms = prefill_run()
        fl = prefill_flops(cfg, PREFILL_TOKENS, layers)
        prefill = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                   "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        # the true 32-bit path, batch 1 (the reference publishes its exact path at batch 1 too)
        del engine
        torch.cuda.empty_cache()
        o32 = EngineOptions(dtype="float32", max_rows=PROMPT, max_full_rows=1, max_slots=2, kv_pages=16, page_size=page, max_context=context)
        e32 = Engine.from_random(cfg, seed=0, options=o32)
        r32, _ = decode_run(e32, 1, 16, 3, 1)
        points["decode_b1_float32"] = round(1000.0 / r32[0][0], 1)
        del e32
        torch.cuda.empty_cache()
        # one request with a long context (bfloat16): where a decode step is mostly the attention over its own cache
        try:
            lms = long_context_run(LONG_CONTEXT)
            points[f"decode_b1_ctx{LONG_CONTEXT}"] = round(1000.0 / lms, 1)
            points[f"hbm_frac_b1_ctx{LONG_CONTEXT}"] = round((weight_bytes + LONG_CONTEXT * kv_token_bytes) / (lms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        except Exception as e:          # the headline line does not hang on this point
            points[f"error_ctx{LONG_CONTEXT}"] = str(e)[:200]
    line = {
        "metric": f"decode tok/s at batch {a.batch} (Llama 3.2 1B shape, 256-token prompts)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)",
        "config": describe(name, cfg, layers, a.batch, page, pk),
        "clocks": clock_info,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 9 * opts.max_rows * 4, "d2h_bytes_per_step": a.batch * 8,
                "how": "LLM.generate: 256-token prompts, 256 outputs, prefill included; generated / wall seconds, median of 3 after one discarded run",
                "engine_steps": stats.steps},
        "gpu_launches": launches * a.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "timed": {"regions": regions, "ms_per_step_of_each": [round(r[0], 4) for r in rs], "reported": "median"},
        "published_elsewhere": "the reference publishes RTX 4090 figures only (2,276 tok/s at batch 8 with prefill time): no vs_baseline",
        "points": points,
    }
    if prefill:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


def serving_shape(a) -> int:
    """The two larger shapes through the scheduler: 3B with 64 requests (prompts of 224 to 288 tokens, 256 outputs);
    8B with 128 requests and a cache pool small enough to force preemption, six of the requests checked against runs alone."""
    import torch
    from stride_b200 import LLM, Engine, EngineOptions

    name, cfg = SHAPES[a.shape]
    cfg = dict(cfg)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers, context, page = cfg["num_hidden_layers"], cfg["max_position_embeddings"], 64
    pk = peaks()
    requests = 64 if a.shape == "3b" else 128
    rng = random.Random(33)
    prompts = [[128000] + [rng.randint(1000, 100000) for _ in range(rng.randint(224, 288) - 1)] for _ in range(requests)]
    need = sum(-(-(len(p) + OUTPUTS) // page) for p in prompts)
    pages = need + requests + 8 if a.shape == "3b" else need * 5 // 8        # 8B: five eighths of what all would hold at the end
    opts = EngineOptions(dtype="bfloat16", max_rows=2048, max_full_rows=requests, max_slots=requests + 1, kv_pages=pages,
                         page_size=page, max_context=context)
    engine = Engine.from_random(cfg, seed=0, options=opts)
    llm = LLM(engine=engine, concurrency=requests, max_rows=2048, prefill_chunk=256)
    clocks = ClockSampler()
    runs = []
    outs = None
    for r in range(3):
        if r == 1:
            clocks.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, max_new_tokens=OUTPUTS)
        dt = time.perf_counter() - t0
        if r > 0:
            runs.append((sum(len(o.tokens) for o in outs) / dt, dt, llm.last_stats))
    clock_info = clocks.stop()
    rate, dt, stats = sorted(runs, key=lambda x: x[0])[len(runs) // 2]
    exact = None
    if a.shape == "8b":
        # the same six requests alone: preemption and replay must not have changed a token or a logit's bits
        solo = LLM(engine=engine, concurrency=1, max_rows=2048, prefill_chunk=256)
        exact = 0
        for i in list(range(0, requests, max(1, requests // 6)))[:6]:
            alone = solo.generate([prompts[i]], max_new_tokens=OUTPUTS, seed=i)[0]
            exact += int(alone.tokens == outs[i].tokens and alone.fingerprint == outs[i].fingerprint)
    kv_token_bytes = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    mean_ctx = sum(len(p) for p in prompts) / requests + OUTPUTS / 2.0
    line = {
        "metric": f"generated tok/s, {requests} requests through the scheduler ({name}, prompts of 224-288 tokens, {OUTPUTS} outputs, prefill included)",
        "value": round(rate, 1), "unit": "tokens/s", "n_gpus": 1, "steps": stats.steps, "warmup": 1, "ms_per_step": round(dt * 1e3 / max(stats.steps, 1), 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)",
        "config": describe(name, cfg, layers, requests, page, pk), "clocks": clock_info,
        "serving": {"requests": requests, "wall_s": round(dt, 3), "engine_steps": stats.steps, "rows": stats.rows, "preemptions": stats.preemptions,
                    "replayed_rows": stats.replayed_rows, "peak_seqs": stats.peak_seqs, "peak_pages": stats.peak_blocks, "pages": pages,
                    "weight_bytes": engine.weight_bytes_per_step(), "kv_bytes_per_token": kv_token_bytes,
                    "decode_step_bytes_at_mean_context": engine.weight_bytes_per_step() + int(requests * mean_ctx * kv_token_bytes)},
    }
    if exact is not None:
        line["serving"]["requests_equal_to_solo_runs"] = f"{exact} of 6"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
