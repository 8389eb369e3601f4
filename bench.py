#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers 36]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the default batch with the
requests' caches filled to the context length: K decode steps (forward pass, logits, sampling)
replayed back to back on the device, timed with CUDA events.  ``e2e`` is the same through the
Python entry point (``Engine.step``): every step copies its inputs from pinned host memory and
reads the sampled tokens back to the host.  ``prefill`` is one 2,048-token prompt through the
step function; ``points`` holds decode at batch 1 and 64.  The engine runs on one GPU; for
--gpus > 1 one line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E2E_SETTLE_STEPS = 24  # untimed engine steps between the prompt phase and the end-to-end warm-up (see measure_decode)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
    max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(raw.get(key), (int, float)):
                    peaks[key] = float(raw[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.process, self.thread = [], None, None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "--id=0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "", 1).isdigit()]
        sm_max = [float(s[1]) for s in self.samples if s[1].replace(".", "", 1).isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(cfg, layers):
    h, i, nq, nkv, d, v = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                           cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer_weights = (nq + 2 * nkv) * d * h + h * nq * d + 2 * i * h + h * i
    return dict(
        layer_weight_elems=per_layer_weights, head_elems=v * h,
        weight_bytes=2 * (layers * per_layer_weights + v * h),      # every weight a decode step uses, once (bf16)
        kv_bytes_per_token=layers * 2 * nkv * d * 2,
        linear_flops_per_token=2 * layers * per_layer_weights,
        attention_flops=lambda tokens: layers * 2 * nq * d * tokens * tokens,  # causal: 2 products over T^2 / 2 pairs
    )


def ideal_seconds(step_log, numbers, cfg, peaks):
    """The least time the logged steps could take on this GPU: every step reads every weight once and the cache of
    the requests in it (bytes / measured copy bandwidth) and multiplies its tokens through the layers and its queries
    with their keys (flops / measured bf16 rate); a step takes the greater of the two, and the steps add up."""
    nq, d, layers = cfg["num_attention_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    total, byte_steps = 0.0, 0
    for step in step_log:
        tokens = sum(count for _, count in step)
        step_bytes = numbers["weight_bytes"] + sum(first + count for first, count in step) * numbers["kv_bytes_per_token"]
        pairs = sum(count * first + count * (count + 1) // 2 for first, count in step)  # (query, key) pairs
        flops = tokens * numbers["linear_flops_per_token"] + 4 * nq * d * layers * pairs + 2 * numbers["head_elems"] * len(step)
        by_bytes, by_flops = step_bytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)
        total += max(by_bytes, by_flops)
        byte_steps += by_bytes >= by_flops
    return total, byte_steps


def generate_workload(which: str) -> int:
    """The serving-style workloads of the larger configurations, end to end through Engine.generate."""
    import torch

    import kirai_b200  # noqa: F401
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.registry import config_from_dict

    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, vocab_size=151936,
                max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0)
    if which == "serving-4b":
        raw = dict(base, num_hidden_layers=36, hidden_size=2560, intermediate_size=9728, num_attention_heads=32,
                   num_key_value_heads=8, tie_word_embeddings=True)
        generator = torch.Generator().manual_seed(3)
        lengths = torch.randint(128, 4097, (64,), generator=generator).tolist()
        new_tokens, temperature = 256, 0.0
        # prompts go in portions of 512 tokens, eight of them to a step beside the tokens of the requests that decode
        options = dict(max_new_tokens=256, max_prefill_tokens=4096, prefill_chunk=512, max_concurrent_requests=64,
                       max_cache_tokens=64 * 4400)
        engine = Engine(config=config_from_dict(raw), random_weights_seed=3, dtype="bfloat16", page_size=16, **options)
    else:
        raw = dict(base, num_hidden_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                   num_key_value_heads=8, tie_word_embeddings=False)
        generator = torch.Generator().manual_seed(4)
        lengths = [8064] * 16
        new_tokens, temperature = 128, 1.0
        options = dict(max_new_tokens=128, max_prefill_tokens=2048, max_concurrent_requests=16, max_cache_tokens=16 * 8256)
        engine = Engine(config=config_from_dict(raw), random_weights_seed=4, dtype="bfloat16", page_size=16, **options)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist() for n in lengths]
    params = SamplingParams(temperature=temperature, seed=7, max_new_tokens=new_tokens, ignore_eos=True)
    peaks, peak_source = load_peaks()
    engine.step_log = []
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    clock_record = clocks.stop()
    generated = sum(len(o.token_ids) for o in outputs)
    stats = engine.stats()
    numbers = model_numbers(raw, raw["num_hidden_layers"])
    ideal, byte_steps = ideal_seconds(engine.step_log, numbers, raw, peaks)
    print(json.dumps({
        "metric": f"generated tokens/s, {which} workload through Engine.generate", "value": generated / seconds,
        "unit": "tokens/s", "n_gpus": 1, "seconds": seconds, "requests": len(prompts), "prompt_tokens": sum(lengths),
        "generated_tokens": generated, "all_tokens_per_s": (sum(lengths) + generated) / seconds, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights", "steps": stats["steps"],
        "graph_steps": stats["graph_steps"], "graphs_captured": len(engine.graphs.graphs), "preemptions": stats["scheduler"]["preemptions"],
        "roofline": {"bound": "per step the greater of bytes / hbm and flops / bf16", "ideal_s": ideal, "measured_s": seconds,
                     "frac": ideal / seconds, "steps_bound_by_bytes": byte_steps, "steps_logged": len(engine.step_log), "of": peak_source,
                     "note": "the measured time holds the graph captures and the host's work between steps"},
        "clocks": clock_record,
        "config": {"model": which, "layers": raw["num_hidden_layers"], "hidden": raw["hidden_size"], "page_size": 16,
                   **{k: v for k, v in options.items()}},
    }))
    return 0


def decode_stamps(batch: int, context: int, layers: int) -> int:
    """Clock stamps of the kernels of one captured decode step: every CTA of the weight-streaming products and of the
    decode attention writes %globaltimer at a few places (csrc/gemm_tcgen05.cu::gemm_stamp, csrc/attention_mma.cu::
    decode_stamp) while a buffer is set.  Prints, per kernel of the second layer, first CTA .. last CTA in us after the
    kernel before had finished.  A measurement aid: the stamps cost a little time themselves."""
    import ctypes

    import torch

    import kirai_b200  # noqa: F401
    from kirai_b200 import Engine
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.registry import config_from_dict

    raw = dict(QWEN3_8B)
    raw["num_hidden_layers"] = layers
    engine = Engine(config=config_from_dict(raw), random_weights_seed=2, dtype="bfloat16", page_size=16, max_new_tokens=512,
                    max_prefill_tokens=2048, max_concurrent_requests=batch, max_cache_tokens=batch * (context + 256))
    runner, cache = engine.runner, engine.runner.cache
    generator = torch.Generator().manual_seed(1)
    requests = [cache.open(i) for i in range(batch)]
    for request in requests:
        prompt = torch.randint(0, raw["vocab_size"], (context - 40,), generator=generator).tolist()
        for first in range(0, len(prompt), 2048):
            runner.step([StepEntry(request, prompt[first : first + 2048], [])], check_errors=False)
    for request in requests:
        assert cache.reserve(request, 32)
    tables = [cache.block_table_array(requests, g) for g in range(len(cache.groups))]
    graph, _ = engine.graphs.get(batch, max(t.shape[1] for t in tables), [r.length + 1 for r in requests])
    graph.load_inputs([1] * batch, [r.length for r in requests], [r.slot for r in requests], tables, [0.0] * batch, [1.0] * batch, [0.0] * batch)
    products = layers * 4 + 1  # per step: q/k/v, o, gate/up, down of every layer, and the output head
    gemm = torch.zeros((2 * products + 2) * 8192, dtype=torch.int64, device="cuda:0")
    attention = torch.zeros((2 * layers + 2) * 8192, dtype=torch.int64, device="cuda:0")
    lib = ops.library()
    lib.kirai_gemm_bf16_set_stamps(ctypes.c_void_p(gemm.data_ptr()))
    lib.kirai_attention_decode_set_stamps(ctypes.c_void_p(attention.data_ptr()))
    graph.capture()  # a warm run, then the capture: the captured launches write to the second half of the buffers
    lib.kirai_gemm_bf16_set_stamps(ctypes.c_void_p(0))
    lib.kirai_attention_decode_set_stamps(ctypes.c_void_p(0))
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    ops.check_device_errors(runner.rt.device)

    def show(name, stamps, columns):
        stamps = stamps[stamps[:, 0] > 0]
        if not len(stamps):
            print(f"{name:10s} no stamps (another kernel variant ran)")
            return
        relative = (stamps - stamps[:, 1].min()) / 1e3
        cells = []
        for index, label in columns:
            seen = relative[:, index][stamps[:, index] > 0]
            if len(seen):
                cells.append(f"{label} {float(seen.min()):6.2f} .. {float(seen.max()):6.2f}")
        print(f"{name:10s} {len(stamps):4d} CTAs | " + " | ".join(cells))

    gemm_columns = [(0, "start"), (2, "first stage"), (3, "products done"), (4, "cluster met"), (6, "tiles summed"), (7, "values stored"), (5, "end")]
    attention_columns = [(0, "start"), (2, "queries in"), (3, "attended"), (4, "merged and stored")]
    per_launch = gemm[products * 8192 :].view(-1, 1024, 8).cpu().double()
    names = ["q/k/v", "o", "gate/up", "down"]
    show("attention", attention[layers * 8192 :].view(-1, 1024, 8).cpu().double()[1], attention_columns)
    for index, name in enumerate(names):
        show(name if index else "q/k/v next", per_launch[4 + (index or 4)], gemm_columns)
    return 0


# ---------------------------------------------------------------------------------------------------------------------
# --workload designs: the Zoferax decoder beside the dense Qwen3 decoder at equal layer sizes
DESIGN_SIZES = {
    # name: width, heads, kv heads, key size, value size, experts, top, expert ff, vocab
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=64, experts=8, top=2, ff=1024, vocab=32000),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, experts=16, top=2, ff=1536, vocab=32000),
}


SILUPEL_LATENT = dict(heads=16, dim=64, rot_dim=64, vdim=64, kv_rank=192)  # a cached row of 256 columns a token
SILUPEL_CHUNK = 1024


def silupel_config(size: dict, layers: int, intermediate: int) -> dict:
    """A Silupel config.json of one size: layers in the order recurrence, attention, latent attention, attention (and
    so on), each with a dense gelu feed-forward as large as the dense model's; attention with the size's heads, half of
    each head rotated (long wavelengths stretched), a soft cap and chunks of 1,024 tokens; the recurrence as wide as
    the model."""
    width = size["width"]
    attention = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"],
                 "scale": size["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": SILUPEL_CHUNK},
                 "rot": {"base": 500000.0, "dims": size["dim"] // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    lat = dict(SILUPEL_LATENT, q_rank=width // 4 + width // 8, scale=(SILUPEL_LATENT["dim"] + SILUPEL_LATENT["rot_dim"]) ** -0.5,
               rot={"base": 10000.0, "dims": SILUPEL_LATENT["rot_dim"]})
    kinds = [("mingru", {"width": width}), ("attention", attention), ("latent_attention", lat), ("attention", attention)]
    mlp = {"kind": "dense", "ff": intermediate}
    return {"architecture": "Silupel", "width": width, "vocab": size["vocab"], "norm": {"eps": 1e-6},
            "layers": [{"type": kinds[i % 4][0], "mixer": dict(kinds[i % 4][1]), "mlp": dict(mlp)} for i in range(layers)]}


FP32_PEAK = 148 * 128 * 2 * 1.965e9  # nominal: 128 32-bit multiply-adds a clock on each of 148 processors at the highest clock


FIGALIX_STATE = dict(vdim=64, state=128, conv=4)   # state-space heads of 64 columns with 128 state rows, inner = 2 width
FIGALIX_MEMORY = dict(dim=128, vdim=256)            # matrix-memory heads, width / 256 of them
FIGALIX_WINDOW = dict(size=1024, keep_first=4)


def figalix_config(size: dict, layers: int, intermediate: int) -> dict:
    """A Figalix config.json of one size: layers in the order state space, side by side (and so on); the state-space
    mixer twice as wide as the model with one group; the attention side with the size's heads, half of each head
    rotated (frequencies stretched by index), a window of 1,024 that keeps four first keys; the memory side with
    width / 256 heads of 128 x 256; feed-forwards in the order dense (as large as the dense model's), experts (the
    size's, with a shared branch as large as one expert)."""
    width = size["width"]
    state = {"heads": 2 * width // FIGALIX_STATE["vdim"], "vdim": FIGALIX_STATE["vdim"], "state": FIGALIX_STATE["state"], "groups": 1,
             "conv": FIGALIX_STATE["conv"], "norm_groups": 1}
    left = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"], "scale": size["dim"] ** -0.5,
            "rot": {"base": 500000.0, "dims": size["dim"] // 2, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}},
            "mask": dict(FIGALIX_WINDOW)}
    right = {"heads": width // 256, "dim": FIGALIX_MEMORY["dim"], "vdim": FIGALIX_MEMORY["vdim"], "gate_cap": 15.0}
    mixers = [("mamba2", state), ("parallel", {"left": left, "right": right})]
    mlps = [{"kind": "dense", "ff": intermediate},
            {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["ff"]}, "shared": {"ff": size["ff"]}}]
    return {"architecture": "Figalix", "width": width, "vocab": size["vocab"], "norm": {"eps": 1e-6}, "residual_mult": 0.5, "logit_softcap": 30.0,
            "layers": [{"type": mixers[i % 2][0], "mixer": dict(mixers[i % 2][1]), "mlp": dict(mlps[i % 2])} for i in range(layers)]}


BIKILIX_LATENT = dict(heads=16, dim=64, rot_dim=64, vdim=64, kv_rank=192)  # a cached row of 256 columns a token
BIKILIX_WINDOW = 1024


def bikilix_config(size: dict, layers: int, intermediate: int) -> dict:
    """A Bikilix config.json of one size: layers in the order latent attention, latent attention, attention, attention
    (and so on); latent attention with 16 heads over a cached row of 256 columns, its rotated part stretched by index;
    attention with the size's heads, a quarter of each head rotated, a window of 1,024; the first layer of four with a
    dense relu^2 feed-forward that holds as many weights as the dense model's gated one, the others with the size's
    experts (clamped gate, two of four groups open); all layers are one pass of a loop, so that the stream is merged
    with the embedding's rows once."""
    width = size["width"]
    attention = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"],
                 "scale": size["dim"] ** -0.5, "mask": {"size": BIKILIX_WINDOW}, "rot": {"base": 1000000.0, "dims": size["dim"] // 4}}
    lat = dict(BIKILIX_LATENT, q_rank=width // 4 + width // 8, scale=(BIKILIX_LATENT["dim"] + BIKILIX_LATENT["rot_dim"]) ** -0.5,
               rot={"base": 500000.0, "dims": BIKILIX_LATENT["rot_dim"],
                    "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}})
    mixers = [("latent_attention", lat), ("latent_attention", lat), ("attention", attention), ("attention", attention)]
    experts = {"kind": "moe", "expert": {"ff": size["ff"], "limit": 7.0},
               "router": {"experts": size["experts"], "top": size["top"], "groups": {"count": 4, "keep": 2}}}
    mlps = [{"kind": "dense", "ff": 3 * intermediate // 2}, experts, experts, experts]
    return {"architecture": "Bikilix", "width": width, "vocab": size["vocab"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [{"type": mixers[i % 4][0], "mixer": dict(mixers[i % 4][1]), "mlp": dict(mlps[i % 4])} for i in range(layers)],
            "loop": {"start": 0, "stop": layers, "times": 1}}


def design_configs(size: dict, layers: int):
    """(Zoferax config.json, Qwen3 config.json, Silupel config.json) of one size: the same width, heads and layer count;
    the dense feed-forward is as large as the experts that one token uses (3 I H = 2 top ff H)."""
    mixer = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["dim"], "vdim": size["vdim"], "scale": size["dim"] ** -0.5}
    mlp = {"kind": "moe", "expert": {"ff": size["ff"]}, "router": {"experts": size["experts"], "top": size["top"]}}
    zoferax = {"architecture": "Zoferax", "width": size["width"], "vocab": size["vocab"], "embedding": {"scale": size["width"] ** 0.5},
               "norm": {"eps": 1e-5}, "layers": [{"type": "attention", "mixer": dict(mixer), "mlp": mlp} for _ in range(layers)]}
    intermediate = -(-(2 * size["top"] * size["ff"]) // (3 * 128)) * 128
    dense = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=size["width"], intermediate_size=intermediate,
                 num_hidden_layers=layers, num_attention_heads=size["heads"], num_key_value_heads=size["kv_heads"],
                 head_dim=size["dim"], vocab_size=size["vocab"], max_position_embeddings=40960, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=False)
    return {"zoferax": zoferax, "qwen3-dense": dense, "silupel": silupel_config(size, layers, intermediate),
            "figalix": figalix_config(size, layers, intermediate), "bikilix": bikilix_config(size, layers, intermediate)}


def _kernel_rows(summary: dict, tokens: int, context_pairs: float, cache_rows: float, size: dict, design: str, peaks,
                 visible=None, requests: int = 1) -> list:
    """One row per entry point of a step: time, the work the DESIGN asks for (not what the kernel chose to compute), and
    that work over the time as a fraction of the measured peak (bytes over the copy bandwidth or flops over the bf16
    rate, whichever is the greater)."""
    import re

    width, heads, kvh, dk = size["width"], size["heads"], size["kv_heads"], size["dim"]
    dv = size["vdim"] if design in ("zoferax", "silupel", "figalix", "bikilix") else dk
    visible = visible or (lambda mask: (context_pairs, cache_rows))
    routed = size["experts"] * size["ff"]
    rows = []
    for name, (count, ms) in sorted(summary.items(), key=lambda item: -item[1][1]):
        flops = bytes_ = simt = 0.0
        label = name
        match = re.search(r"m=(\d+) n=(\d+) k=(\d+) form=(\d+)", name)
        if match and "grouped" in name and design == "bikilix" and int(match.group(2)) == BIKILIX_LATENT["vdim"] \
                and int(match.group(3)) == BIKILIX_LATENT["kv_rank"] + BIKILIX_LATENT["rot_dim"]:
            # the heads' value matrices as groups over rows laid out head by head: the design's work is kv_rank columns a head
            h_, k_, n_ = BIKILIX_LATENT["heads"], BIKILIX_LATENT["kv_rank"], BIKILIX_LATENT["vdim"]
            flops = 2.0 * tokens * h_ * k_ * n_ * count
            bytes_ = (tokens * h_ * (2.0 * k_ + 4.0 * n_) + 2.0 * h_ * k_ * n_) * count
            label += " (a product per head, heads as groups)"
        elif match and "grouped" in name:
            # rows sorted by expert: the design's work is tokens * top rows through one expert's matrices each
            m, n, k, form = map(int, match.groups())
            rows_used = tokens * size["top"]
            flops = 2.0 * rows_used * n * k * count
            bytes_ = (2.0 * rows_used * (k + n) + 2.0 * size["experts"] * n * k) * count
            label += " (experts, rows sorted by expert)"
        elif match:
            m, n, k, form = map(int, match.groups())
            flops, bytes_ = 2.0 * m * n * k, 2.0 * (m * k + n * k) + m * (n // 2 if form == 2 else n) * (4 if form in (1, 3) else 2)
            if design in ("zoferax", "bikilix") and (routed in (n, k) or 2 * routed == n):  # the experts: a token needs top of them
                share = size["top"] / size["experts"]
                flops *= share
                bytes_ = 2.0 * m * k * (share if k == routed else 1) + 2.0 * n * k * min(1.0, share * max(1, m)) + m * n * 2.0 * (share if n == routed else 2)
                label += " (experts; work = the chosen experts')"
            flops, bytes_ = flops * count, bytes_ * count
        elif "attention" in name and "heads=" in name:
            # a launch that says its shape: pairs and cache rows of the keys that its mask lets a query see
            a_heads, a_kv, a_d, a_mask = (int(v) for v in re.search(r"heads=(\d+) kv=(\d+) d=(\d+) mask=(-?\d+)", name).groups())
            pairs, rows_read = visible(a_mask)
            shared = 1.0 if (design in ("silupel", "bikilix") and a_kv == 1) else 2.0  # a latent row is key and value in one
            flops = 2.0 * a_heads * 2 * a_d * pairs * count
            bytes_ = (2.0 * a_kv * shared * a_d * rows_read + 2.0 * tokens * a_heads * 2 * a_d) * count
        elif "attention" in name:
            flops = 2.0 * heads * (dk + dv) * context_pairs * count
            bytes_ = (2.0 * kvh * (dk + dv) * cache_rows + 2.0 * tokens * heads * (dk + dv)) * count
        elif "head_major" in name or "head_gate_rows" in name:
            bytes_ = tokens * BIKILIX_LATENT["heads"] * (4.0 * (BIKILIX_LATENT["kv_rank"] + BIKILIX_LATENT["rot_dim"]) if "major" in name
                                                          else 10.0 * BIKILIX_LATENT["vdim"]) * count
        elif "head_linear_gate" in name:
            # a product per head between the attention over the shared latent and the output projection, and the gate
            t_, h_, k_, n_ = (int(v) for v in re.search(r"t=(\d+) heads=(\d+) k=(\d+) n=(\d+)", name).groups())
            flops = 2.0 * t_ * h_ * k_ * n_ * count
            bytes_ = (2.0 * t_ * h_ * (k_ + n_) + 4.0 * t_ * h_ * n_ + 2.0 * h_ * k_ * n_) * count
        elif "add_bias" in name:
            bytes_ = tokens * width * 8.0 * count
        elif "norm_add_norm" in name:
            bytes_ = tokens * width * 14.0 * count
        elif "stream_copy" in name:
            bytes_ = tokens * width * 6.0 * count
        elif "kirai_relu2_" in name and "gate" not in name:
            bytes_ = tokens * size.get("intermediate", width) * 3 // 2 * 4.0 * count
        elif "ssm_walk" in name or "matrix_memory_walk" in name:
            # a walk: every token touches the whole state of every head once (decay, outer product, read-out), in 32-bit
            # on the ordinary pipe; a request's state is read and written once a step
            if "ssm" in name:
                cells = (2 * width // FIGALIX_STATE["vdim"]) * FIGALIX_STATE["vdim"] * FIGALIX_STATE["state"]
                cols = 2 * width + 2 * FIGALIX_STATE["state"] + 2 * width // FIGALIX_STATE["vdim"] + 2 * width
            else:
                cells = (width // 256) * FIGALIX_MEMORY["dim"] * FIGALIX_MEMORY["vdim"]
                cols = (width // 256) * (2 * FIGALIX_MEMORY["dim"] + 2 * FIGALIX_MEMORY["vdim"] + 2)
            simt = 6.0 * tokens * cells * count
            bytes_ = (4.0 * tokens * cols + 8.0 * cells * requests) * count
        elif "ssm_chunks" in name or "matrix_memory_chunks" in name:
            # chunks of 64 tokens: a token meets the chunk's earlier tokens (scores over the state's rows, weighted values) and
            # the carried state twice (read-out, the chunk's share of the update), in 32-bit on the ordinary pipe
            if "ssm" in name:
                s_heads, s_d, s_dv = 2 * width // FIGALIX_STATE["vdim"], FIGALIX_STATE["state"], FIGALIX_STATE["vdim"]
                cols = 2 * width + 2 * FIGALIX_STATE["state"] + 2 * width // FIGALIX_STATE["vdim"] + 2 * width
            else:
                s_heads, s_d, s_dv = width // 256, FIGALIX_MEMORY["dim"], FIGALIX_MEMORY["vdim"]
                cols = (width // 256) * (2 * FIGALIX_MEMORY["dim"] + 2 * FIGALIX_MEMORY["vdim"] + 2)
            simt = tokens * s_heads * (64.0 * (s_d + s_dv) + 4.0 * s_d * s_dv) * count
            bytes_ = (4.0 * tokens * cols + 8.0 * s_heads * s_d * s_dv * requests) * count
        elif "conv_silu" in name:
            bytes_ = tokens * (2 * width + 2 * FIGALIX_STATE["state"]) * 8.0 * count
        elif "gated_group_norm" in name:
            bytes_ = tokens * 2 * width * 10.0 * count
        elif "rms_pair_mean" in name:
            bytes_ = tokens * width * 12.0 * count
        elif "add_dyt" in name or "add_scaled" in name:
            bytes_ = tokens * width * 16.0 * count
        elif "head_gate" in name:
            bytes_ = tokens * heads * dv * 4.0 * count
        elif "gated_expert_gate" in name:
            bytes_ = tokens * routed * 6.0 * count
        elif "qkv_wide_norm" in name:
            cols = heads * dk + kvh * (dk + dv)
            bytes_ = tokens * (4.0 * cols + 2.0 * cols) * count
        elif "qk_norm_rope" in name:
            bytes_ = tokens * 2.0 * (2 * (heads + kvh) * dk + 2 * kvh * dk) * count
        elif "add_layernorm" in name:
            bytes_ = tokens * width * 14.0 * count
        elif "token_shift" in name:
            bytes_ = tokens * width * 6.0 * count
        elif "mingru" in name:
            bytes_ = tokens * width * 14.0 * count
        elif "qkv_rope_write" in name or "latent_prepare" in name:
            bytes_ = tokens * 6.0 * (heads * dk + kvh * (dk + dv)) * count
        elif "sigmoid_gate" in name:
            bytes_ = tokens * heads * dv * 8.0 * count
        elif "gated_activation" in name and design == "bikilix":
            bytes_ = tokens * size["top"] * size["ff"] * 6.0 * count  # the chosen experts' rows: gate and up in, hidden out
        elif "gated_activation" in name:
            bytes_ = tokens * size.get("intermediate", width) * 6.0 * count
        elif "norm_add" in name:
            bytes_ = tokens * width * 14.0 * count
        elif "add_rmsnorm" in name:
            bytes_ = tokens * width * 12.0 * count
        elif "route_" in name:
            bytes_ = tokens * size["top"] * width * 4.0 * count
        elif "relu2_gate" in name:
            bytes_ = tokens * routed * 4.0 * count
        elif "router" in name:
            bytes_ = (tokens * width * 2.0 + size["experts"] * width * 4.0) * count
        elif "embedding" in name or "round_rows" in name:
            bytes_ = tokens * width * 6.0 * count
        seconds = ms / 1e3
        ideal = {"bytes": bytes_ / (peaks["hbm_gbs"] * 1e9), "flops": flops / (peaks["bf16_tflops"] * 1e12), "fp32": simt / FP32_PEAK}
        bound = max(ideal, key=ideal.get)
        frac = ideal[bound] / seconds if seconds > 0 else 0.0
        rows.append({"kernel": label, "launches": count, "ms": round(ms, 4), "frac_of_measured_peak": round(frac, 3), "bound": bound})
    return rows


def compare_designs(args) -> int:
    """Prefill and decode throughput of the Zoferax design and of the dense Qwen3 decoder at equal layer sizes, random
    weights, and each step's time by entry point with its fraction of the measured peaks.  Prints one JSON line."""
    import torch

    import kirai_b200  # noqa: F401
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.registry import config_from_dict

    peaks, peak_source = load_peaks()
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    T, R, context, layers = args.prefill_tokens, args.batch, args.context, (8 if args.layers == QWEN3_8B["num_hidden_layers"] else args.layers)
    torch.cuda.set_device(0)
    generator = torch.Generator().manual_seed(99)
    clocks = ClockSampler()
    clocks.start()
    out = {}
    for size_name in [s for s in args.sizes.split(",") if s]:
        size = DESIGN_SIZES[size_name]
        size = dict(size, intermediate=-(-(2 * size["top"] * size["ff"]) // (3 * 128)) * 128)
        configs = design_configs(size, layers)
        for design in [d for d in args.designs.split(",") if d]:
            raw = configs[design]
            vocab = size["vocab"]
            engine = Engine(config=config_from_dict(raw), random_weights_seed=3, dtype="bfloat16", page_size=args.page_size,
                            max_new_tokens=4 * (warmup + steps) + 64, max_prefill_tokens=T, max_concurrent_requests=R,
                            max_cache_tokens=(2 * R + 2) * (context + 256))
            runner = engine.runner

            def prompt(n):
                return torch.randint(0, vocab, (n,), generator=generator).tolist()

            # prefill: one prompt of T tokens through the step function
            times = []
            for it in range(warmup + 5):
                pages = runner.cache.open(("prefill", it))
                tokens = prompt(T)
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([StepEntry(pages, tokens, [T - 1])], check_errors=False)
                stop.record()
                torch.cuda.synchronize()
                if it >= warmup:
                    times.append(start.elapsed_time(stop))
                runner.cache.close(pages)
            prefill_ms = statistics.median(times)
            pages = runner.cache.open(("prefill", "timed"))
            with ops.launch_timer() as timer:
                runner.step([StepEntry(pages, prompt(T), [T - 1])], check_errors=False)
            def seen(p, mask):
                # how many keys position p sees: its chunk's, all up to itself, or its window's and the kept first ones
                if mask < 0:
                    return p % -mask + 1
                if mask == 0:
                    return p + 1
                window, kept = mask & ((1 << 20) - 1), mask >> 20
                return min(p + 1, window) + max(0, min(kept, p + 1 - window))

            def prefill_visible(mask):
                # pairs of (query, key it sees) and key rows read, for a prompt of T tokens from position 0
                return float(sum(seen(p, mask) for p in range(T))), float(T)

            def decode_visible(mask):
                return R * float(seen(context + 1, mask)), R * float(seen(context + 1, mask))

            prefill_kernels = _kernel_rows(timer.summary(), T, T * (T + 1) / 2.0, T, size, design.split("-")[0], peaks, prefill_visible)
            runner.cache.close(pages)
            # decode: R requests at the context length; through Engine.step (captured steps, host tokens in and out)
            params = SamplingParams(temperature=0.0, max_new_tokens=4 * (warmup + steps) + 64, ignore_eos=True)
            requests = [engine.add_request(prompt(context), params) for _ in range(R)]
            while any(r.pending > 1 or not r.output for r in requests):
                engine.step()
            for _ in range(warmup + 8):
                engine.step()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            decode_ms = (time.perf_counter() - t0) / steps * 1e3
            engine.drain()
            for r in requests:
                engine.scheduler.abort(r)
            # the same step's kernels one by one: an eager step of R single tokens on caches filled to the context
            held = [runner.cache.open(("decode", i)) for i in range(R)]
            for request in held:
                runner.step([StepEntry(request, prompt(context), [])], check_errors=False)
            runner.step([StepEntry(request, prompt(1), [0]) for request in held], check_errors=False)
            with ops.launch_timer() as timer:
                runner.step([StepEntry(request, prompt(1), [0]) for request in held], check_errors=False)
            decode_kernels = _kernel_rows(timer.summary(), R, R * (context + 2.0), R * (context + 2.0), size, design.split("-")[0], peaks,
                                          decode_visible, requests=R)
            ops.check_device_errors(runner.rt.device)
            out[f"{size_name}/{design}"] = {
                "prefill_tokens_per_s": T / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
                "decode_tokens_per_s": R / (decode_ms / 1e3), "decode_ms_per_step": decode_ms,
                "captured_decode_steps": engine.counters.get("graph_steps", 0),
                "prefill_kernels": prefill_kernels, "decode_kernels": decode_kernels,
            }
            del engine, runner, held, requests
            torch.cuda.empty_cache()
    line = {"metric": f"prefill and decode tokens/s of {args.designs} at equal layer sizes", "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights (seed 3)",
            "config": {"sizes": {k: DESIGN_SIZES[k] for k in args.sizes.split(",") if k}, "layers": layers, "prefill_tokens": T,
                       "decode_batch": R, "context": context, "page_size": args.page_size, "peaks": peak_source,
                       "l2": "every size's weights and cache exceed L2"},
            "results": out, "clocks": clocks.stop()}
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a power of two)")
    parser.add_argument("--points", default="1,64", help="other decode batches to measure (comma separated, '' for none)")
    parser.add_argument("--no-check", action="store_true",
                        help="skip the check of the captured decode step against the step function before each timing")
    parser.add_argument("--workload", default="decode", choices=["decode", "serving-4b", "batch-32b", "decode-stamps", "designs"],
                        help="decode: the default measurement, whose one JSON line the driver reads.  serving-4b: 64 requests with prompts of "
                             "128..4096 tokens, 512-token prefill portions mixed with decode, 256 new tokens each, greedy, "
                             "Qwen3-4B shape.  batch-32b: 16 requests of 8,064 prompt tokens, 128 new tokens at temperature 1, "
                             "Qwen3-32B shape.  Both run through Engine.generate and print their own one line.  decode-stamps: "
                             "the kernels' own clock stamps inside one captured decode step (--batch, --context, --layers; "
                             "4 layers are enough), a table instead of the JSON line.  designs: prefill and decode of the "
                             "designs named by --designs (default: the Zoferax decoder beside the dense Qwen3 decoder) at "
                             "equal layer sizes (--sizes), with every step's time by kernel; a line of its own.")
    parser.add_argument("--sizes", default="2k,4k", help="layer sizes of --workload designs: " + ", ".join(DESIGN_SIZES))
    parser.add_argument("--designs", default="zoferax,qwen3-dense",
                        help="which designs --workload designs measures, comma separated: zoferax, silupel, figalix, bikilix, qwen3-dense")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "michaelasper/kir-ai is a Rust workspace (no setup.py or pyproject.toml, "
                          "pip install refuses it) and its GPU path is Apple Metal; no Rust toolchain or Metal device here"}))
        return 0
    if args.gpus != 1:
        print("bench.py measures one GPU: the engine is a single-GPU engine by design (--gpus 1)")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.workload == "designs":
        return compare_designs(args)
    if args.workload == "decode-stamps":
        return decode_stamps(args.batch, args.context, min(args.layers, 4) if args.layers == QWEN3_8B["num_hidden_layers"] else args.layers)
    if args.workload != "decode":
        return generate_workload(args.workload)

    import torch

    import kirai_b200
    from kirai_b200 import Engine, SamplingParams
    from kirai_b200.csrc import ops
    from kirai_b200.engine.batch import StepEntry
    from kirai_b200.registry import config_from_dict

    raw = dict(QWEN3_8B)
    raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    numbers = model_numbers(raw, args.layers)
    peaks, peak_source = load_peaks()
    batches = [args.batch] + [int(b) for b in args.points.split(",") if b.strip()]
    max_batch = max(batches)
    page_size = args.page_size
    context = args.context
    torch.cuda.set_device(0)
    # what a request may generate while the others are still being filled, and while it is warmed up and timed twice
    new_token_cap = max_batch * -(-context // args.prefill_tokens) + 4 * (warmup + steps) + E2E_SETTLE_STEPS + 64
    engine = Engine(config=config, random_weights_seed=2, dtype="bfloat16", page_size=page_size,
                    max_new_tokens=new_token_cap, max_prefill_tokens=args.prefill_tokens, max_concurrent_requests=max_batch,
                    max_cache_tokens=max_batch * (context + 256))
    runner = engine.runner
    generator = torch.Generator().manual_seed(1234)

    def random_prompt(n):
        return torch.randint(0, raw["vocab_size"], (n,), generator=generator).tolist()

    clocks = ClockSampler()
    clocks.start()

    # ------------------------------------------------------------------ prefill: one prompt through the step function
    T = args.prefill_tokens
    prefill_times = []
    for it in range(warmup + 5):
        pages = runner.cache.open(("prefill", it))
        prompt = random_prompt(T)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(pages, prompt, [T - 1])], check_errors=False)
        stop.record()
        torch.cuda.synchronize()
        if it >= warmup:
            prefill_times.append(start.elapsed_time(stop))
        runner.cache.close(pages)
    ops.check_device_errors(runner.rt.device)
    prefill_ms = statistics.median(prefill_times)
    prefill_flops = numbers["linear_flops_per_token"] * T + numbers["attention_flops"](T) + 2 * numbers["head_elems"]
    prefill = {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "flops": prefill_flops}

    # ------------------------------------------------------------------ decode
    checks = {}

    def check_decode(batch):
        """What is timed below, checked first: on `batch` requests filled to the context length, the captured decode
        step and the step queued behind it give the logits of the step function on the same cache state."""
        from kirai_b200.engine.graphs import captured_and_eager_logits

        cache = runner.cache
        requests = [cache.open(("check", batch, i)) for i in range(batch)]
        filled = context - 8
        for request in requests:
            prompt = random_prompt(filled)
            for first in range(0, filled, args.prefill_tokens):
                runner.step([StepEntry(request, prompt[first : first + args.prefill_tokens], [])], check_errors=False)
        result = captured_and_eager_logits(engine.graphs, requests, random_prompt(batch))
        worst, scale = 0.0, 0.0
        for captured, eager in zip(result["captured"], result["eager"]):
            if not bool(torch.isfinite(captured).all()) or not bool(torch.isfinite(eager).all()):
                raise SystemExit(f"check failed at batch {batch}: logits are not finite")
            worst = max(worst, float((captured - eager).abs().max()))
            scale = max(scale, float(eager.abs().max()))
        for request in requests:
            cache.close(request)
        ops.check_device_errors(runner.rt.device)
        if worst > 0.02 * scale:  # the bound of the bfloat16 tests
            raise SystemExit(f"check failed at batch {batch}: captured and eager logits differ by {worst} (largest logit {scale})")
        checks[batch] = {"max_abs_diff": worst, "largest_logit": scale}

    def measure_decode(batch):
        """Fills `batch` requests' caches through the engine, then times decode steps two ways."""
        if not args.no_check:
            check_decode(batch)
        # Requests that finish their prompt early decode while the others are still being filled, one
        # token per fill step; start them that much lower so that all end near the context length.
        budget = args.prefill_tokens
        fill_steps = batch * -(-context // budget)
        filled = max(16, context - (2 * (warmup + steps) + 4 + E2E_SETTLE_STEPS) - fill_steps)
        params = SamplingParams(temperature=0.0, max_new_tokens=new_token_cap, ignore_eos=True)
        requests = [engine.add_request(random_prompt(filled), params) for _ in range(batch)]
        while any(r.pending > 1 or not r.output for r in requests):
            engine.step()  # prompt portions under the token budget, then the first sampled tokens
        # (a) through the Python entry point: host tokens in and out every step.  The prompt phase just before ran
        # under the power cap; the clocks take about ten decode steps to come back (4.05 falling to 3.65 ms a step
        # at 8 requests), so a fixed number of steps settles them before the warm-up steps that the caller asked for.
        for _ in range(E2E_SETTLE_STEPS + warmup):
            engine.step()
        torch.cuda.synchronize()
        launches_before = engine.counters["graph_steps"]
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - t0
        assert engine.counters["graph_steps"] - launches_before == steps
        engine.drain()  # the engine queues decode steps one ahead
        # (b) on the device: the captured step feeds itself; pages for the steps ahead are reserved first
        ahead = warmup + steps
        for r in requests:
            assert runner.cache.reserve(r.pages, ahead + 1)
        cache = runner.cache
        tables = [cache.block_table_array([r.pages for r in requests], g) for g in range(len(cache.groups))]
        # the captured step that the engine itself would replay for these requests (its choice of attention kernel)
        graph, fresh = engine.graphs.get(batch, max(t.shape[1] for t in tables), [r.pages.length + 1 for r in requests])
        graph.load_inputs([r.token_at(r.computed) for r in requests], [r.pages.length for r in requests],
                          [r.pages.slot for r in requests], tables, [0.0] * batch, [1.0] * batch, [0.0] * batch)
        if fresh:
            graph.capture()
        lengths_before = sum(r.pages.length for r in requests) / batch
        for _ in range(warmup):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        device_ms = start.elapsed_time(stop) / steps
        ops.check_device_errors(runner.rt.device)
        mean_context = lengths_before + warmup + steps / 2.0
        step_bytes = numbers["weight_bytes"] + batch * mean_context * numbers["kv_bytes_per_token"]
        result = dict(batch=batch, device_ms=device_ms, tokens_per_s=batch / (device_ms / 1e3),
                      e2e_tokens_per_s=batch * steps / e2e_seconds, e2e_ms=e2e_seconds / steps * 1e3,
                      bytes=step_bytes, gbs=step_bytes / (device_ms / 1e3) / 1e9, context=mean_context,
                      kernels=graph.kernels_per_replay, h2d=graph.ahead_input_bytes, d2h=4 * batch + 4)
        for r in requests:
            engine.scheduler.abort(r)
        return result

    results = {b: measure_decode(b) for b in batches}

    # a second denominator: what a kernel that only reads reaches here (2 GiB, fresh for every pass: above L2)
    ceiling = None
    try:
        scratch = torch.empty(2 << 30, dtype=torch.uint8, device="cuda:0")
        scratch.fill_(1)
        for _ in range(3):
            ops.stream_read(scratch)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(5):
            ops.stream_read(scratch)
        stop.record()
        torch.cuda.synchronize()
        ops.check_device_errors(runner.rt.device)
        ceiling = 5 * scratch.numel() / (start.elapsed_time(stop) / 1e3) / 1e9
        del scratch
    except (RuntimeError, AttributeError):
        pass
    clock_record = clocks.stop()
    main_result = results[args.batch]
    roofline = {"bound": "hbm", "achieved": main_result["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": main_result["gbs"] / peaks["hbm_gbs"], "of": peak_source}
    if ceiling:
        # the copy figure counts a read and a write; a read-only stream goes faster, and the decode step only reads
        roofline["read_only_ceiling"] = ceiling
        roofline["frac_of_read_only_ceiling"] = main_result["gbs"] / ceiling
    line = {
        "metric": "decode tok/s at batch 8 (points: batch 1 and 64); prefill tok/s at 2,048 tokens (Qwen3-8B)",
        "value": main_result["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_result["device_ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights (seed 2)",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_of_config": QWEN3_8B["num_hidden_layers"],
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "global_batch": args.batch, "seq_len": context, "context_at_timing": round(main_result["context"]),
            "page_size": page_size, "prefill_tokens": T, "parallelism": "single GPU",
            "l2": "weights (16 GB) and cache exceed L2; no flush needed", "peaks": peak_source,
        },
        "prefill": {k: prefill[k] for k in ("value", "tokens", "ms", "frac")},
        "roofline": roofline,
        "points": {f"decode_b{b}": results[b]["tokens_per_s"] for b in batches if b != args.batch},
        "points_detail": {f"decode_b{b}": {"ms": results[b]["device_ms"], "gbs": results[b]["gbs"],
                                           "frac": results[b]["gbs"] / peaks["hbm_gbs"],
                                           "e2e": results[b]["e2e_tokens_per_s"]} for b in batches},
        "e2e": {"value": main_result["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": main_result["e2e_ms"],
                "h2d_bytes_per_step": main_result["h2d"], "d2h_bytes_per_step": main_result["d2h"],
                "settle_steps": E2E_SETTLE_STEPS},
        "gpu_launches": main_result["kernels"] * steps,
        "clocks": clock_record,
        "checked": bool(checks) and all(b in checks for b in batches),
        "check": {f"decode_b{b}": checks[b] for b in checks},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
