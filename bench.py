"""Headline benchmark: Qwen3-0.6B batch-1 greedy decode at long context.

Workload (one "step"): reset, prefill a 2048-token uniform-random prompt, then
256 greedy decode steps on seed-0 random-init bf16 weights of the Qwen3-0.6B
architecture.  `value` is decode tokens/s with everything resident in HBM (the
256-step device-resident chain timed with CUDA events); `e2e` is decode
tokens/s through the public decoder API with host inputs and outputs
(`decode_steps(first_token:int, n) -> cpu tensor`), and the prefill through
`prefill_step(cpu ids)` is reported beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With --gpus N > 1 (under torchrun) every rank runs an independent replica on
its own GPU with its own prompt; there is no data-path communication.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from megaqwen_b200.spec import QWEN3_0_6B  # noqa: E402
from megaqwen_b200.synthetic import random_prompt, random_weights  # noqa: E402

PROMPT_LEN = 2048
NEW_TOKENS = 256
MAX_SEQ = 2320            # position + steps must stay below max_seq_len (the reference's bound)
METRIC = "decode_tokens_per_s_b1_ctx2048"
WORKLOAD = "qwen3-0.6b random-init bf16, batch 1, 2048-token random prompt + 256 greedy decode steps"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        # nvidia-smi numbers GPUs physically; with CUDA_VISIBLE_DEVICES set the CUDA ordinal is
        # another GPU, so the device is named by its UUID
        try:
            self.index = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
        except Exception:
            self.index = str(index)
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop_evt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for n, v in zip(names, out[2:]):
                    if v.strip().lower() == "active":
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=5)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


from megaqwen_b200.replicas import aggregate_throughput, barrier, dist_env, init_control_plane, max_over_ranks  # noqa: E402


# DRAM bytes of one decode step from a recorded ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum) at the cache length below; NOT re-measured by this run.
NCU_STEP_DRAM_BYTES = 1430.2e6
NCU_STEP_CACHE_LEN = 2050
NCU_CAPTURE = "per-phase kernels at commit a2e3ddb; the persistent kernel streams a repacked copy of the same bytes"


def host_threads() -> int:
    """Host cores this process may run on."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference(sample_new: int, threads: int | None = None):
    """The reference's HF bf16 path on the host cores: decode tokens/s at context
    2048 on a bounded sample (2048-token prompt, `sample_new` new tokens)."""
    from oracle.hf_reference import build_hf_model, time_hf_decode
    torch.set_num_threads(threads or host_threads())
    w = random_weights(QWEN3_0_6B, MAX_SEQ)
    model = build_hf_model(QWEN3_0_6B, w)
    prompt = random_prompt(QWEN3_0_6B, PROMPT_LEN, 2, 0)
    tps, prefill_s = time_hf_decode(model, prompt, sample_new)
    return tps, prefill_s, torch.get_num_threads()


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    sample_new = 64
    vals, pre = [], []
    from oracle.hf_reference import build_hf_model, time_hf_decode
    torch.set_num_threads(host_threads())   # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core it may
    w = random_weights(QWEN3_0_6B, MAX_SEQ)
    model = build_hf_model(QWEN3_0_6B, w)
    prompt = random_prompt(QWEN3_0_6B, PROMPT_LEN, 2, 0)
    for i in range(args.warmup + args.steps):
        tps, prefill_s = time_hf_decode(model, prompt, sample_new)
        if i >= args.warmup:
            vals.append(tps)
            pre.append(prefill_s)
    v = sum(vals) / len(vals)
    cores = torch.get_num_threads()
    sample = f"{PROMPT_LEN}-token prompt + {sample_new} greedy single-token forwards per step (timed directly), HF Qwen3ForCausalLM bf16 on CPU"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sample_new / v,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "prefill_tokens_per_s": PROMPT_LEN / (sum(pre) / len(pre)),
        "host_cpus": os.cpu_count(),
    }))


def measure_other_configs(dev, w, only_config5=False, seq_seed0=0):
    """The remaining BASELINE configurations on one GPU (reported beside the headline):
    config 3 (1024-token prefill + 32 steps), config 4 (batch 32, ragged 256-512 prompts,
    128 steps) and config 5 (batch 64, 1024-token prompts, 256 steps)."""
    from megaqwen_b200.batch import MegakernelBatchDecoder
    from megaqwen_b200.decoder import MegakernelDecoder
    from megaqwen_b200.synthetic import random_lengths
    spec = QWEN3_0_6B
    out = {}
    lw = [t.to(dev) for t in w["layer_weights"]]
    embed = w["embed_weight"].to(dev)
    common = (embed, lw, w["final_norm_weight"].to(dev), embed)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    if only_config5:
        return _measure_batched(out, common, w, dev, only_config5, seq_seed0)
    # config 3
    dec = MegakernelDecoder(*common, w["cos_table"].to(dev), w["sin_table"].to(dev), spec.num_layers, MAX_SEQ, 1024)
    prompt = random_prompt(spec, 1024, 3, 0).to(dev)
    best = 1e9
    for _ in range(4):
        dec.reset()
        torch.cuda.synchronize(dev)
        e0, e1 = events()
        e0.record(); tok = dec.prefill_step(prompt); e1.record()
        torch.cuda.synchronize(dev)
        best = min(best, e0.elapsed_time(e1))
    dec._chain(tok, 32, True)                                  # builds the graph
    dec.position_ = 1024
    torch.cuda.synchronize(dev)
    e0, e1 = events()
    e0.record(); dec._chain(tok, 32, True); e1.record()
    torch.cuda.synchronize(dev)
    out["config3_prefill1024"] = {"prefill_ms": best, "prefill_tokens_per_s": 1024 / best * 1e3,
                                  "prefill_tflops": spec.prefill_flops(1024) / best / 1e9,
                                  "decode32_tokens_per_s": 32 / e0.elapsed_time(e1) * 1e3}
    del dec
    torch.cuda.empty_cache()

    return _measure_batched(out, common, w, dev, only_config5, seq_seed0)


def _measure_batched(out, common, w, dev, only_config5, seq_seed0):
    from megaqwen_b200.batch import MegakernelBatchDecoder
    from megaqwen_b200.synthetic import random_lengths
    spec = QWEN3_0_6B

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def batched(name, lens, steps, max_seq, cfg_idx, kv_fp8=False):
        B = len(lens)
        cos, sin = w["cos_table"][:max_seq].contiguous().to(dev), w["sin_table"][:max_seq].contiguous().to(dev)
        bd = MegakernelBatchDecoder(*common, cos, sin, spec.num_layers, max_seq, B, max(lens), kv_fp8=kv_fp8)
        prompts = [random_prompt(spec, n, cfg_idx, seq_seed0 + i) for i, n in enumerate(lens)]
        bd.prefill_batch(prompts)                              # untimed: first-use set-up (kernel attributes, tensor maps, staging buffers)
        bd.reset()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        first = bd.prefill_batch(prompts)
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        chunk = 32
        bd.decode_batch_steps(first, chunk)                    # builds the graph
        bd._positions[:B].copy_(torch.tensor(lens, dtype=torch.int32))
        torch.cuda.synchronize(dev)
        e0, e1 = events()
        e0.record()
        cur, done = first, 0
        while done < steps:
            o = bd.decode_batch_steps(cur, chunk)
            cur = o[-1]
            done += chunk
        e1.record()
        torch.cuda.synchronize(dev)
        bd.check_status()
        ms = e0.elapsed_time(e1)
        mean_len = sum(lens) / B + steps / 2
        # bytes a step must move: the weights once, every cached K/V row once (half as many with the e4m3 shadow)
        step_bytes = spec.weight_bytes() + B * spec.kv_bytes_per_position() * (mean_len + 1) * (0.5 if kv_fp8 else 1.0)
        out[name] = {"batch": B, "prefill_tokens_per_s": sum(lens) / (t1 - t0), "decode_tokens_per_s": B * steps / ms * 1e3,
                     "ms_per_step": ms / steps, "achieved_GBps": step_bytes / (ms / steps * 1e-3) / 1e9}
        del bd
        torch.cuda.empty_cache()

    if not only_config5:
        batched("config4_batch32_ragged", random_lengths(32, 256, 512), 128, 1024, 4)
    batched("config5_batch64_ctx1024", [1024] * 64, 256, 1296, 5)
    if not only_config5:
        # the same workload with the attention reading the e4m3 shadow KV cache (opt-in, row f3)
        batched("config5_batch64_ctx1024_kv_fp8", [1024] * 64, 64, 1296, 5, kv_fp8=True)
    return out


def decode_by_context(dec, dev, peak):
    """Batch-1 decode latency at fixed cache lengths (32 steps starting at each length, over the
    cache the headline run left behind): microseconds per token and the fraction of the HBM
    roofline for the bytes of those steps, for the graph-replayed per-phase kernels and for the
    persistent kernel (one cooperative launch)."""
    out = {}
    keep = dec.use_persistent
    for L in (1, 16, 128, 512, 1024, 2048):
        nbytes = sum(QWEN3_0_6B.decode_bytes(L + i) for i in range(32)) / 32
        row = {}
        for name, persistent in (("graph", False), ("persistent", True)):
            if persistent and not dec.persistent_available:
                continue
            dec.use_persistent = persistent
            best = 1e9
            for _ in range(3):
                dec.position_ = L - 1          # the step writes position L-1 and attends over L entries
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); dec._chain(17, 32, True); e1.record()
                torch.cuda.synchronize(dev)
                best = min(best, e0.elapsed_time(e1) / 32 * 1e3)
            gbs = nbytes / (best * 1e-6) / 1e9
            row[name] = {"us_per_token": best, "achieved_GBps": gbs, "frac": gbs / peak, "frac_of_8TBps": gbs / 8000.0}
        out[str(L)] = row
    dec.use_persistent = keep
    dec.check_status()
    return out


def parity_check(dec):
    """The headline workload's first 64 decode steps, teacher-forced, against the committed HF
    bf16 CPU fixture (tests/golden/full_cfg2_p2048_n256.npz; rank 0's prompt is that prompt)."""
    import numpy as np
    z = np.load(os.path.join(ROOT, "tests", "golden", "full_cfg2_p2048_n256.npz"))

    def f32(a):
        return torch.from_numpy(a.astype(np.uint16).view(np.int16).copy()).view(torch.bfloat16).float()

    n = 64
    tokens = z["tokens"].tolist()
    dec.reset()
    tok0, lg = dec.prefill_step_logits(torch.from_numpy(z["prompt"]))
    rows, got = [lg.cpu()], [tok0]
    for t in tokens[:n - 1]:
        tok, l2 = dec.decode_step_logits(int(t))
        rows.append(l2.cpu()); got.append(tok)
    lgs = torch.stack(rows)
    top_idx = torch.from_numpy(z["top_idx"][:n]).long()
    d = torch.cat([(lgs[:, ::64] - f32(z["strided"][:n])).abs().flatten(),
                   (torch.gather(lgs, 1, top_idx) - f32(z["top_vals"][:n])).abs().flatten()])
    return {"against": "HF Qwen3ForCausalLM bf16 CPU fixture, 2048-token prompt, 64 teacher-forced steps (every 64th logit + HF's top-8)",
            "max_abs": float(d.max()), "mean_abs": float(d.mean()), "frac_within_2e-2": float((d <= 2e-2).float().mean()),
            "tokens_identical": sum(int(a == b) for a, b in zip(got, tokens[:n])), "tokens_compared": n}


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = init_control_plane(world)
    from megaqwen_b200.decoder import MegakernelDecoder

    w = random_weights(QWEN3_0_6B, MAX_SEQ)
    lw = [t.to(dev) for t in w["layer_weights"]]
    embed = w["embed_weight"].to(dev)
    dec = MegakernelDecoder(embed, lw, w["final_norm_weight"].to(dev), embed, w["cos_table"].to(dev),
                            w["sin_table"].to(dev), QWEN3_0_6B.num_layers, MAX_SEQ, PROMPT_LEN)
    prompt = random_prompt(QWEN3_0_6B, PROMPT_LEN, 2, rank).pin_memory()
    chunk = args.chunk
    dec.use_persistent = bool(args.persistent)

    def one_step(timed: bool):
        """Returns (decode_ms_device, decode_ms_e2e, prefill_ms_e2e, launches)."""
        dec.reset()
        torch.cuda.synchronize(dev)
        l0 = dec.launches
        t0 = time.perf_counter()
        first = dec.prefill_step(prompt)
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        # (a) device-resident chain, CUDA events on the launching stream
        pos0 = dec.position()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first_dev = torch.tensor([first], dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        l1 = dec.launches
        ev0.record()
        done = 0
        cur = first_dev
        while done < NEW_TOKENS:
            n = min(chunk, NEW_TOKENS - done)
            out = dec._chain(cur, n, True)
            cur = out[n - 1:n].clone()
            done += n
        ev1.record()
        torch.cuda.synchronize(dev)
        l2 = dec.launches
        dev_ms = ev0.elapsed_time(ev1)
        dec.check_status()
        # (b) the same 256 steps through the public API with host in/out
        dec.position_ = pos0
        torch.cuda.synchronize(dev)
        t2 = time.perf_counter()
        toks = dec.decode_steps(first, NEW_TOKENS)
        t3 = time.perf_counter()
        assert toks.numel() == NEW_TOKENS and not toks.is_cuda
        return dev_ms, (t3 - t2) * 1e3, (t1 - t0) * 1e3, l2 - l1

    for _ in range(args.warmup):
        one_step(False)
    barrier(dist)
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(local)
    sampler.start()
    dev_ms, e2e_ms, pre_ms, launches = [], [], [], 0
    wall0 = time.perf_counter()
    for _ in range(args.steps):
        a, b, c, l = one_step(True)
        dev_ms.append(a); e2e_ms.append(b); pre_ms.append(c); launches += l
    torch.cuda.synchronize(dev)
    barrier(dist)
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    tot_dev, tot_e2e, tot_pre = max_over_ranks(dist, [sum(dev_ms), sum(e2e_ms), sum(pre_ms)])
    other = None
    if args.other_configs:
        # Every rank measures the batched configurations on its own GPU (config 5 is the replica
        # configuration: batch 64 x 1024-token prompts x 256 steps per GPU); the aggregate uses the
        # slowest rank's time.  Only N = 1 also runs configs 3 and 4.
        try:
            other = measure_other_configs(dev, w, only_config5=(world > 1), seq_seed0=64 * rank)
            ms5 = other["config5_batch64_ctx1024"]["ms_per_step"]
            (worst_ms5,) = max_over_ranks(dist, [ms5])
            other["config5_replicas"] = {"n_gpus": world, "batch_per_gpu": 64, "prompt_len": 1024, "decode_steps": 256,
                                         "ms_per_step_max_over_ranks": worst_ms5,
                                         "aggregate_decode_tokens_per_s": world * 64 / worst_ms5 * 1e3}
        except Exception as exc:
            other = {"error": repr(exc)[:200]}
            max_over_ranks(dist, [0.0])
    if rank != 0:
        return
    n_tok = NEW_TOKENS * args.steps * world
    value = aggregate_throughput(NEW_TOKENS * args.steps, world, tot_dev / 1e3)
    e2e = aggregate_throughput(NEW_TOKENS * args.steps, world, tot_e2e / 1e3)
    peak, peak_kind = load_peaks()
    # algorithmic bytes of the decode steps of one pass: cache length after step i is 2048 + i + 1
    bytes_pass = sum(QWEN3_0_6B.decode_bytes(PROMPT_LEN + i + 1) for i in range(NEW_TOKENS))
    step_s = (tot_dev / 1e3) / (NEW_TOKENS * args.steps)
    achieved = bytes_pass / NEW_TOKENS / step_s / 1e9
    # DRAM traffic of one step: a RECORDED ncu capture at cache length 2050 (read + write 1430.2 MB
    # against 1427.3 MB algorithmic), moved to this run's mean cache length with the per-position
    # KV bytes (traffic grows in proportion to them); this run does not measure it
    mean_len = PROMPT_LEN + (NEW_TOKENS + 1) / 2
    traffic = NCU_STEP_DRAM_BYTES + (mean_len - NCU_STEP_CACHE_LEN) * (QWEN3_0_6B.decode_bytes(2) - QWEN3_0_6B.decode_bytes(1))
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": tot_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"{world} independent replica(s), no communication",
                   "l2": "inputs larger than L2 (1.19 GB of weights stream per token)", "steps_per_launch": chunk},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * NEW_TOKENS + 4,
                "prefill_tokens_per_s": PROMPT_LEN * args.steps * world / (tot_pre / 1e3),
                "prefill_h2d_bytes_per_step": 4 * PROMPT_LEN},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_kind": "recorded",
                     "traffic_source": "recorded ncu capture (dram__bytes_read.sum + dram__bytes_write.sum of one step at cache length 2050: "
                                       + NCU_CAPTURE + "), scaled to the mean cache length of this run; not re-measured here",
                     "algorithmic_bytes": bytes_pass / NEW_TOKENS,
                     "peak_kind": peak_kind,
                     "kernel": ("k_decode_stream: one persistent launch per chunk of decode steps; per-step figures = launch / steps"
                                if args.persistent else "one decode step of the per-phase kernels (141 PDL-chained launches, graph replay)"),
                     "frac_of_8TBps": achieved / 8000.0, "us_per_token": step_s * 1e6},
        "clocks": clocks,
        "wall_s": wall,
    }
    if args.other_configs and world == 1:
        try:
            line["parity"] = parity_check(dec)
        except Exception as exc:
            line["parity"] = {"error": repr(exc)[:200]}
        try:
            line["decode_by_context"] = decode_by_context(dec, dev, peak)
        except Exception as exc:
            line["decode_by_context"] = {"error": repr(exc)[:200]}
    if args.other_configs:
        line["other_configs"] = other
    if not args.no_cpu and world == 1:
        try:
            tps, prefill_s, cores = cpu_reference(64)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "reference",
                                    "sample": f"{PROMPT_LEN}-token prompt + 64 greedy single-token forwards timed directly, HF Qwen3ForCausalLM bf16 on CPU",
                                    "prefill_tokens_per_s": PROMPT_LEN / prefill_s}
        except Exception as exc:  # the baseline is reported, never a gate
            line["cpu_baseline"] = {"value": None, "error": repr(exc)[:200]}
    print(json.dumps(line))


def run_ncu_case(args):
    """Small case for profiler captures: a few eager decode steps at context 2048
    over a cache filled with random values (no 2048-step prompt before them)."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from megaqwen_b200.decoder import MegakernelDecoder
    w = random_weights(QWEN3_0_6B, MAX_SEQ)
    embed = w["embed_weight"].to(dev)
    dec = MegakernelDecoder(embed, [t.to(dev) for t in w["layer_weights"]], w["final_norm_weight"].to(dev), embed,
                            w["cos_table"].to(dev), w["sin_table"].to(dev), QWEN3_0_6B.num_layers, MAX_SEQ, PROMPT_LEN)
    if args.ncu_batch > 0:
        from megaqwen_b200.batch import MegakernelBatchDecoder
        del dec
        B = args.ncu_batch
        bd = MegakernelBatchDecoder(embed, [t.to(dev) for t in w["layer_weights"]], w["final_norm_weight"].to(dev), embed,
                                    w["cos_table"].to(dev), w["sin_table"].to(dev), QWEN3_0_6B.num_layers, MAX_SEQ, B, 64)
        first = random_prompt(QWEN3_0_6B, B, 5, 0)
        bd.batch_ = B                      # no prefill: the caches are filled with random values below
        bd.k_cache_.normal_(0, 1)
        bd.v_cache_.normal_(0, 1)
        bd._positions[:B].fill_(args.ncu_pos)
        out = bd.decode_batch_steps(first, args.ncu_case, use_graph=False)
        torch.cuda.synchronize(dev)
        bd.check_status()
        print(json.dumps({"ncu_batch": B, "steps": args.ncu_case, "position": args.ncu_pos, "tokens": out[-1][:4].tolist()}))
        return
    if args.ncu_prefill > 0:
        prompt = random_prompt(QWEN3_0_6B, args.ncu_prefill, 3, 0)
        tok = None
        for _ in range(args.ncu_case):
            dec.reset()
            tok = dec.prefill_step(prompt)
        torch.cuda.synchronize(dev)
        print(json.dumps({"ncu_prefill_tokens": args.ncu_prefill, "repeats": args.ncu_case, "next_token": tok}))
        return
    dec.k_cache_.normal_(0, 1)
    dec.v_cache_.normal_(0, 1)
    dec.position_ = args.ncu_pos
    if args.ncu_persistent:
        toks = dec.decode_steps_cuda_persistent(17, args.ncu_case)
    else:
        toks = dec.decode_steps_cuda(17, args.ncu_case)
    torch.cuda.synchronize(dev)
    dec.check_status()
    print(json.dumps({"ncu_case_steps": args.ncu_case, "position": dec.position(), "tokens": toks.tolist()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunk", type=int, default=32, help="decode steps per CUDA graph (per launch with --persistent)")
    ap.add_argument("--persistent", action="store_true",
                    help="time the persistent kernel (one cooperative launch per chunk) instead of the graph-replayed per-phase kernels")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-other-configs", dest="other_configs", action="store_false",
                    help="skip the extra single-GPU measurements of configs 3-5")
    ap.add_argument("--ncu-case", type=int, default=0, help="run N eager decode steps at --ncu-pos and exit (profiler case)")
    ap.add_argument("--ncu-pos", type=int, default=PROMPT_LEN)
    ap.add_argument("--ncu-prefill", type=int, default=0, help="profiler case: N prefills of this many tokens instead of decode steps")
    ap.add_argument("--ncu-batch", type=int, default=0, help="profiler case: batched decode steps with this batch size")
    ap.add_argument("--ncu-persistent", action="store_true", help="profiler case runs the persistent chain kernel")
    args = ap.parse_args()
    if args.ncu_case > 0:
        run_ncu_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
