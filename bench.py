#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B-shape Q4_K GGUF decode throughput (batch 64, plus batch 1 and the
2048-token prefill TTFT as side metrics) on N B200 GPUs of one node, tensor-parallel for N > 1.

    python bench.py --gpus N --steps K --warmup W

Weights are seeded N(0, 0.02) quantized to Q4_K (embeddings / output Q6_K); prompts are uniform
random ids; there is no dataset or checkpoint involved.  A "step" is one decode step of the whole
batch.  The device-timed value replays the engine's self-advancing decode graph (real
autoregression: each step consumes the previous step's arg-max); the end-to-end value calls the
public ``engine.decode`` once per step with the step's inputs copied from pinned host memory and
the sampled ids read back.

``vs_baseline`` is this run's value over the same benchmark served by plain PyTorch on the same GPUs right after it
(``baseline/llama_torch.py``: weights dequantized to bf16, ``torch.matmul``, fused SDPA, NCCL all-reduce, CUDA graph);
``--impl baseline`` runs only that arm.  ``--impl reference`` reports why the reference repository cannot be run.
``extra`` also carries the training (GPT-2-small, 3 + 3 steps) and expert-parallel MoE decode throughput on the same
GPUs, unless ``--extras none``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import threading
import time

MODEL = "llama-3-8b-shape"
PROMPT_LEN = 2048
BATCH = 64


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled from a thread
    every 20 ms (a timed region can be shorter than one ``nvidia-smi -lms`` period), with one sample
    taken at the start and one at the end in any case.  Reading only; no setting is touched."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int):
        self.idx, self.sm, self.mask, self.max_mhz = gpu_index, [], 0, None
        self.h = self.nv = self.thread = None
        self.running = False

    def _sample(self):
        try:
            self.sm.append(float(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
            try:
                self.mask |= int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:
                self.mask |= int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
        except Exception:
            pass

    def _loop(self):
        while self.running:
            self._sample()
            time.sleep(0.02)

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            return
        self._sample()
        self.running = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["not_measured"], "samples": 0}
        self._sample()
        self.running = False
        self.thread.join(timeout=1)
        reasons = sorted(n for n, bit in self.REASONS.items() if self.mask & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


def reference_arm():
    # The reference tree is a TypeScript/Rust monorepo without a Python project or any ML engine:
    # a pip install of that tree stops with "Neither 'setup.py' nor 'pyproject.toml' found".
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference has no installable Python package and no inference/training engine "
                                     "(pip: neither setup.py nor pyproject.toml found)"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; marks the run invalid)")
    ap.add_argument("--extras", default="train,moe", help="side benchmarks reported under extra: comma list of train, moe, or none")
    ap.add_argument("--no-baseline", action="store_true", help="skip the PyTorch baseline arm (vs_baseline stays null)")
    ap.add_argument("--tp", type=int, default=0, help="ranks per tensor-parallel replica (0: all ranks up to 4; 8 GPUs then run "
                    "two replicas of 4, each serving half of the batch)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.impl not in ("b200", "baseline"):
        raise SystemExit("--impl is one of b200, baseline, reference")
    K, W = args.steps, max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from openagents_b200.models.config import PRESETS
    from openagents_b200.models.engine import LlamaEngine, PAGE
    from openagents_b200.models.qweight import RandomSource
    from openagents_b200.models.weights import PLAN_Q4_K

    cfg = PRESETS[args.model]
    valid = True
    if args.layers:
        cfg = cfg.with_(n_layers=args.layers)
        valid = False
    B, P = args.batch, args.prompt_len
    # Layout: ``dp`` replicas of ``tp`` ranks.  A replica shards the model (tensor parallel, this package's fused kernels
    # over the symmetric heap) and serves B / dp of the sequences; replicas never talk to each other.  Beyond four ranks
    # the per-layer all-reduce latency outweighs what a thinner weight shard saves for a model of this size, so eight
    # GPUs run as two replicas of four unless --tp says otherwise.
    tp = args.tp if args.tp > 0 else (world if world <= 4 else 4)
    if world % tp or B % (world // tp):
        raise SystemExit(f"--tp {tp} does not divide {world} ranks / batch {B}")
    dp = world // tp
    tp_rank, replica, Bl = rank % tp, rank // tp, B // dp
    layout = f"tp{tp}" if dp == 1 else (f"dp{dp}" if tp == 1 else f"dp{dp}xtp{tp}")
    tp_group = None
    if world > 1 and dp > 1 and tp > 1:
        for r0 in range(0, world, tp):          # every rank creates every group, in the same order
            grp = dist.new_group(list(range(r0, r0 + tp)))
            if r0 == replica * tp:
                tp_group = grp
    comm = None
    if tp > 1:    # symmetric heap: the fp32 residual stream and the bf16 all-gathered activations of a prefill chunk
        from openagents_b200.parallel.tp import TPComm
        comm = TPComm(tp_rank, tp, dev, heap_bytes=(4 * P + tp) * cfg.d_model * 6 + (64 << 20), group=tp_group)
    total_steps = 2 * (K + W) + 8
    max_ctx = P + total_steps + PAGE
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab, (B + 1, P), generator=g)
    extra_prompt = prompts[B]
    my_prompts = prompts[replica * Bl:(replica + 1) * Bl]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def baseline_arm(with_clocks: bool):
        from baseline.llama_torch import run_decode_baseline
        return run_decode_baseline(cfg, RandomSource(cfg, PLAN_Q4_K, 0, dev), dev, tp_rank, tp, Bl, P, K, W, my_prompts, barrier,
                                   max_over_ranks, ClockSampler(local) if with_clocks else None, group=tp_group, total_batch=B)

    if args.impl == "baseline":
        r = baseline_arm(True)
        if rank == 0:
            print(json.dumps({"impl": "baseline", "metric": f"llama3_8b_q4k_decode_tok_s_bs{B}", "value": round(r["value"], 1),
                              "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(r["ms_per_step"], 4),
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": 1.0, "dtype": "bf16", "data": "synthetic",
                              "config": {"model": cfg.name, "weights": "the product run's Q4_K/Q6_K weights dequantized to bf16",
                                         "global_batch": B, "seq_len": P, "kv_cache": "contiguous bf16", "parallelism": layout,
                                         "stack": "torch.matmul (cuBLAS) + SDPA + NCCL all-reduce + CUDA graph", "valid": valid},
                              "clocks": r["clocks"],
                              "e2e": {"value": round(r["e2e_value"], 1), "unit": "tokens/s", "ms_per_step": round(r["e2e_ms_per_step"], 4),
                                      "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
                              "gpu_launches": 0, "extra": {"weight_bytes_per_gpu": r["weight_bytes_per_gpu"]}}))
        if world > 1:
            dist.destroy_process_group()
        return
    # The model is served from a GGUF FILE: rank 0 writes the seeded Q4_K / Q6_K tensors once (standard block bytes, this
    # package's C++ writer), every rank then opens the file with the C++ reader and loads its shard from it.
    gguf_path, gguf_write_s, src, weights_from = None, None, None, "gguf file"
    try:
        import tempfile
        from openagents_b200.gguf import GGUFWriter
        from openagents_b200.models.qweight import GGUFSource
        from openagents_b200.models.weights import tensor_specs
        gguf_path = os.path.join(tempfile.gettempdir(), f"b200_bench_{cfg.name}_{cfg.n_layers}l_q4k.gguf")
        if rank == 0 and not os.path.exists(gguf_path):
            tw = time.time()
            rs = RandomSource(cfg, PLAN_Q4_K, 0, dev)
            wr = GGUFWriter(gguf_path + ".tmp")
            for k_, v_ in cfg.to_gguf_metadata().items():
                wr.add_meta(k_, v_)
            for spec in tensor_specs(cfg):
                r_ = rs.get(spec.name)
                wr.add_tensor_raw(spec.name, int(r_.type), spec.shape, r_.data.cpu().numpy())
            wr.write()
            os.replace(gguf_path + ".tmp", gguf_path)
            gguf_write_s = time.time() - tw
        barrier()
        src = GGUFSource(gguf_path, dev)
    except Exception as e:      # noqa: BLE001 - no room for the file, read-only temp dir, ...: generate the same tensors in memory
        weights_from = f"generated in memory ({type(e).__name__}: {e})"[:160]
        if world > 1:
            dist.barrier()
        src = RandomSource(cfg, PLAN_Q4_K, 0, dev)
    t0 = time.time()
    eng = LlamaEngine(cfg, src, device=dev, max_batch=Bl + 1, max_ctx=max_ctx,
                      max_tokens=4 * P, tp_rank=tp_rank, tp_world=tp, comm=comm)
    load_s = time.time() - t0

    # ---- prefill TTFT: one 2048-token prompt, device time of the whole forward incl. first arg-max
    X = Bl                                                    # the extra sequence used for time-to-first-token and batch 1
    eng.begin(X)
    eng.forward_tokens([X], [extra_prompt[:64].tolist()])    # warm the kernels on a short chunk
    eng.end(X)
    ttft = []
    for rep in range(3):
        eng.begin(X)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _, nxt1 = eng.forward_tokens([X], [extra_prompt.tolist()])
        e1.record()
        barrier()
        ttft.append(max_over_ranks(e0.elapsed_time(e1)))
        if rep < 2:
            eng.end(X)
    ttft_ms = min(ttft[1:])

    # ---- batch prefill (untimed): 4 sequences per call
    first = []
    for b0 in range(0, Bl, 4):
        ids = list(range(b0, min(Bl, b0 + 4)))
        for i in ids:
            eng.begin(i)
        _, nxt = eng.forward_tokens(ids, [my_prompts[i].tolist() for i in ids])
        first += nxt.tolist()
    eng.check_status()

    gpu_index = local
    # ---- bs1 decode (sequence B, already prefilled)
    tok1 = [int(nxt1[0].item())]
    last = eng.decode_steps([X], tok1, W)[W - 1].clone()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = {0: e0}
    eng.decode_steps([X], [int(last[0].item())], K, on_replay=lambda i: marks[i].record() if i in marks else None)
    e1.record()
    barrier()
    bs1_ms = max_over_ranks(e0.elapsed_time(e1)) / K
    launches_bs1 = eng.launches_per_decode

    # ---- bs64 decode: device-timed, self-advancing graph
    seqs = list(range(Bl))
    hist = eng.decode_steps(seqs, first, W)
    last = hist[W - 1].tolist()
    sampler = ClockSampler(gpu_index)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = {0: e0}
    hist = eng.decode_steps(seqs, last, K, on_replay=lambda i: marks[i].record() if i in marks else None)
    e1.record()
    barrier()
    clocks = sampler.stop()
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / K
    launches = eng.launches_per_decode * K
    last = hist[K - 1].tolist()
    eng.check_status()

    # ---- bs64 decode end to end through engine.decode(): per step H2D of the inputs, D2H of the ids
    for _ in range(W):
        _, nxt = eng.decode(seqs, last)
        last = nxt.tolist()
    barrier()
    h2d_before = eng.h2d_bytes
    t_start = time.perf_counter()
    for _ in range(K):
        _, nxt = eng.decode(seqs, last)
        last = nxt.tolist()                    # device -> host read of the step's result
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t_start) * 1e3) / K
    h2d = (eng.h2d_bytes - h2d_before) // K        # counted by the engine from the tensors it copies: ids, pos, slot,
                                                   # lengths every step, page-table rows when a sequence takes a new page
    h2d, d2h = h2d * world, 4 * Bl * world         # every rank copies its replica's inputs in and reads the ids back
    eng.check_status()

    # ---- N > 1, side measurement: the same global batch served by N independent replicas (whole model per GPU,
    # B / N sequences each), the configuration a model that fits one GPU would be deployed in for throughput.
    # The headline stays the tensor-parallel number; a failure here is reported, not raised.
    replicas = None
    if tp > 1 and B % world == 0 and cfg.d_model <= 4096:
        Br, rep_ms, err = B // world, -1.0, ""
        try:                       # local work only in here: a rank that fails must not leave the others in a collective
            rep = LlamaEngine(cfg, RandomSource(cfg, PLAN_Q4_K, 0, dev), device=dev, max_batch=Br, max_ctx=max_ctx,
                              max_tokens=P, tp_rank=0, tp_world=1, comm=None)
            firsts = []
            for i in range(Br):
                rep.begin(i)
                _, nx = rep.forward_tokens([i], [prompts[rank * Br + i].tolist()])
                firsts += nx.tolist()
            ids_l = list(range(Br))
            h = rep.decode_steps(ids_l, firsts, W)
            lastl = h[W - 1].tolist()
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            marks = {0: r0}
            rep.decode_steps(ids_l, lastl, K, on_replay=lambda i: marks[i].record() if i in marks else None)
            r1.record()
            torch.cuda.synchronize()
            rep.check_status()
            rep_ms = r0.elapsed_time(r1) / K
            del rep
        except Exception as e:      # noqa: BLE001 - a side measurement must not take the benchmark down
            err = f"{type(e).__name__}: {e}"[:200]
        t = torch.tensor([rep_ms, -rep_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)                 # slowest rank, and whether any rank failed
        slowest, any_failed = float(t[0].item()), float(t[1].item()) > 0
        replicas = ({"error": err or "a rank failed"} if any_failed else
                    {"decode_tok_s": round(B / (slowest * 1e-3), 1), "ms_per_step": round(slowest, 4), "batch_per_gpu": Br,
                     "parallelism": f"dp{world} (independent replicas)"})

    weight_bytes = eng.weight_bytes()
    scratch_bytes = eng.scratch_bytes()
    launches_per_step = eng.launches_per_decode
    del eng
    if comm is not None:
        del comm
    import gc
    gc.collect()
    torch.cuda.empty_cache()

    # ---- the same benchmark on plain PyTorch (cuBLAS + SDPA + NCCL), same GPUs, same weights: the baseline arm
    base, base_err = None, None
    if not args.no_baseline:
        try:
            base = baseline_arm(False)
        except Exception as e:      # noqa: BLE001 - the product number stands even if the comparison arm fails
            base_err = f"{type(e).__name__}: {e}"[:200]
        gc.collect()
        torch.cuda.empty_cache()

    # ---- side benchmarks on the same GPUs: training throughput and expert-parallel MoE decode
    extras = {} if args.extras == "none" else {k: None for k in args.extras.split(",") if k}
    if "train" in extras:
        try:
            import bench_train
            r = bench_train.run(3, 3)
            extras["train"] = None if r is None else {"train_tok_s": r["value"], "train_ms_per_step": r["ms_per_step"],
                                                      "train_model_tflops_per_gpu": r["extra"]["model_tflops_per_gpu"],
                                                      "train_vs_torch_arm": r["vs_baseline"], "train_torch_arm": r["extra"]["baseline"],
                                                      "train_config": r["config"]}
        except Exception as e:      # noqa: BLE001
            extras["train"] = {"train_error": f"{type(e).__name__}: {e}"[:200]}
        gc.collect()
        torch.cuda.empty_cache()
    if "moe" in extras:
        try:
            import bench_moe
            margs = argparse.Namespace(gpus=world, steps=16, warmup=4, batch=256, prefill=4096, context=4096, layers=0)
            r = bench_moe.run(margs)
            extras["moe"] = None if r is None else {"moe_decode_tok_s": r["value"], "moe_ms_per_step": r["ms_per_step"],
                                                    "moe_prefill_tok_s": r["extra"]["prefill_tok_s"], "moe_config": r["config"]}
        except Exception as e:      # noqa: BLE001
            extras["moe"] = {"moe_error": f"{type(e).__name__}: {e}"[:200]}
        gc.collect()
        torch.cuda.empty_cache()

    if rank == 0:
        value = B / (dev_ms * 1e-3)
        out = {
            "metric": f"{cfg.name.replace('-shape', '').replace('-', '_').replace('llama_3', 'llama3')}_q4k_decode_tok_s_bs{B}", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None if base is None else round(value / base["value"], 4), "dtype": "bf16",
            "data": "synthetic",
            "config": {"model": cfg.name, "weights": "Q4_K (embeddings/output Q6_K), seeded N(0,0.02)",
                       "global_batch": B, "seq_len": P, "decode_context": f"{P}+", "kv_cache": "paged fp16, 16-token pages",
                       "parallelism": layout, "batch_per_replica": Bl, "l2": "inputs larger than L2 (weights + KV cache >> 126 MB)",
                       "valid": valid},
            "clocks": clocks,
            "e2e": {"value": round(B / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "extra": {"decode_tok_s_bs1": round(1.0 / (bs1_ms * 1e-3), 1), "ms_per_step_bs1": round(bs1_ms, 4),
                      "launches_per_step_bs1": launches_bs1, "prefill_ttft_ms": round(ttft_ms, 3),
                      "prefill_tok_s": round(P / (ttft_ms * 1e-3), 1), "load_s": round(load_s, 1), "weights_from": weights_from,
                      "gguf_file_bytes": os.path.getsize(gguf_path) if gguf_path and os.path.exists(gguf_path) else None,
                      "gguf_write_s": None if gguf_write_s is None else round(gguf_write_s, 1),
                      "weight_bytes_per_gpu": weight_bytes, "prefill_scratch_bytes_per_gpu": scratch_bytes,
                      "launches_per_step_bs64": launches_per_step,
                      "baseline": ({"error": base_err} if base is None else
                                   {"decode_tok_s": round(base["value"], 1), "ms_per_step": round(base["ms_per_step"], 4),
                                    "e2e_tok_s": round(base["e2e_value"], 1), "weight_bytes_per_gpu": base["weight_bytes_per_gpu"],
                                    "stack": "torch.matmul (cuBLAS) + SDPA + NCCL all-reduce + CUDA graph"}),
                      **{k: v for e in extras.values() if e for k, v in e.items()},
                      **({"replicas": replicas} if replicas else {})},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
