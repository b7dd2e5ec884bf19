"""End-to-end workloads for the BASELINE.json configs that are not the headline (bench.py runs the headline, config #2):

    --workload fastgen70b   config #5  Llama-2-70B shapes, FastGen ragged batching, tensor parallel over all ranks (TP = world),
                                       bf16 or block-scaled fp8 (--quant wf8af8_mx | wf8af8_block | wf8af8), synthetic ragged arrivals
    --workload mixtral      config #4  Mixtral 8x7B shapes, expert parallel over all ranks, ZeRO-2 training step
    --workload ulysses13b   config #3  Llama-2-13B shapes, Ulysses sequence parallel over all ranks, ZeRO-3, --seq-len tokens total

Launched like bench.py (`python -m torch.distributed.run ... bench.py --workload X --gpus N ...`).  Random-init weights, synthetic
tokens.  Every timed region is end to end: the step's inputs start in pinned host memory, the step's result (sampled tokens /
loss) is read back to the host; timing = CUDA events on the device, max over ranks, barrier + synchronize on both sides.  Rank 0
prints one JSON line in the bench.py vocabulary.  `--layers L` cuts the depth for shake-down runs (the model name then says so)."""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))


def _timed(torch, dist, fn, steps, warmup):
    """-> (ms per call of fn, max over ranks, device-timed), clocks dict (rank 0)."""
    from bench import ClockSampler
    dev = torch.device("cuda", torch.cuda.current_device())
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    if dist.get_rank() == 0:
        sampler.start()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([a.elapsed_time(b)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if dist.get_rank() == 0 else None
    return ms.item() / steps, clocks


def _line(metric, value, unit, world, args, ms, config, clocks, launches, extra):
    out = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic tokens (uniform random ids), random-init weights", "impl": "own", "config": config,
           "gpu_launches": launches, "clocks": clocks}
    out.update(extra)
    return out


# ------------------------------------------------------------------------------------------------ config #5: FastGen 70B
class _LazyLlamaState(dict):
    """HF-named Llama state dict whose tensors are drawn on the device when they are asked for (a 70B checkpoint is 140 GB; the
    engine's loader shards and drops every tensor as soon as its parameter is complete)."""

    def __init__(self, cfg, device, dtype):
        super().__init__()
        self.cfg, self.device, self.dtype = cfg, device, dtype

    def items(self):
        import torch
        c = self.cfg
        h, inter, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
        d = h // c["num_attention_heads"]
        hq, hkv = c["num_attention_heads"], c["num_key_value_heads"]

        def r(*shape, std=0.02, one=False):
            t = torch.empty(*shape, device=self.device, dtype=self.dtype).normal_(0.0, std)
            return t + 1 if one else t

        yield "model.embed_tokens.weight", r(V, h)
        for i in range(c["num_hidden_layers"]):
            p = f"model.layers.{i}."
            yield p + "self_attn.q_proj.weight", r(hq * d, h)
            yield p + "self_attn.k_proj.weight", r(hkv * d, h)
            yield p + "self_attn.v_proj.weight", r(hkv * d, h)
            yield p + "self_attn.o_proj.weight", r(h, hq * d)
            yield p + "input_layernorm.weight", r(h, one=True)
            yield p + "post_attention_layernorm.weight", r(h, one=True)
            yield p + "mlp.gate_proj.weight", r(inter, h)
            yield p + "mlp.up_proj.weight", r(inter, h)
            yield p + "mlp.down_proj.weight", r(h, inter)
        yield "model.norm.weight", r(h, one=True)
        yield "lm_head.weight", r(V, h)


def run_fastgen70b(args):
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.inference.v2 import RaggedInferenceEngineConfig, build_engine_from_state_dict
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    L = args.layers or 80
    cfg = dict(vocab_size=32000, hidden_size=8192, intermediate_size=28672, num_hidden_layers=L, num_attention_heads=64,
               num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=4096)
    n_seqs, budget, gen = args.sequences, args.token_budget, args.gen_tokens
    g = torch.Generator().manual_seed(7)
    prompt_lens = torch.randint(args.prompt_min, args.prompt_max + 1, (n_seqs, ), generator=g).tolist()
    max_ctx = max(prompt_lens) + gen * (args.steps + args.warmup) + 8
    blocks = n_seqs * (-(-max_ctx // 128) + 1) + 8
    ecfg = RaggedInferenceEngineConfig(tensor_parallel={"tp_size": world},
                                       state_manager={"max_ragged_batch_size": budget, "max_ragged_sequence_count": max(n_seqs, 8),
                                                      "max_tracked_sequences": max(n_seqs, 8), "max_context": -(-max_ctx // 128) * 128,
                                                      "memory_config": {"mode": "allocate", "size": blocks}},
                                       quantization={"quantization_mode": args.quant})
    t_build = time.perf_counter()
    eng = build_engine_from_state_dict("llama", cfg, _LazyLlamaState(cfg, dev, torch.bfloat16), ecfg, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    prompts = [torch.randint(0, cfg["vocab_size"], (n, ), generator=g).pin_memory() for n in prompt_lens]
    uids = list(range(n_seqs))
    state = {"next": None, "first": True}

    def prefill():
        """Ragged arrivals: every forward takes whole prompts while they fit the token budget, then the next prompt's head as a
        chunk (split-fuse); the unfinished prompt continues in the next forward."""
        for u in uids:
            if not state["first"]:
                eng.flush(u)
        state["first"] = False
        nxt = torch.zeros(n_seqs, dtype=torch.long)
        pos = [0] * n_seqs
        i = 0
        forwards = 0
        while i < n_seqs:
            batch_u, batch_t, room = [], [], budget
            j = i
            while j < n_seqs and room > 0 and len(batch_u) < ecfg.state_manager.max_ragged_sequence_count:
                take = min(room, prompt_lens[j] - pos[j])
                batch_u.append(j)
                batch_t.append(prompts[j][pos[j]:pos[j] + take])
                pos[j] += take
                room -= take
                if pos[j] < prompt_lens[j]:
                    break
                j += 1
            logits = eng.put(batch_u, batch_t)
            tok = logits.argmax(-1).cpu()  # device -> host: the sampled tokens
            for k, u in enumerate(batch_u):
                if pos[u] == prompt_lens[u]:
                    nxt[u] = tok[k]
            forwards += 1
            i = j
        state["next"] = nxt
        return forwards

    def decode():
        nxt = state["next"]
        for _ in range(gen):
            logits = eng.put(uids, [nxt[u:u + 1] for u in uids])
            nxt = logits.argmax(-1).cpu()
        state["next"] = nxt

    l0 = native.launch_count
    ms_prefill, _ = _timed(torch, dist, prefill, 1, 1)  # one untimed pass (allocations, tensor maps), one timed
    ms_decode, clocks = _timed(torch, dist, decode, args.steps, args.warmup)
    launches = native.launch_count - l0
    if rank == 0:
        prompt_tokens = sum(prompt_lens)
        ctx = sum(prompt_lens) / n_seqs + gen * (args.warmup + args.steps / 2)
        ops = eng._model._tp_ops() if hasattr(eng._model, "_tp_ops") else None
        extra = {
            "prefill": {"prompt_tokens": prompt_tokens, "ms": round(ms_prefill, 2), "tokens_per_s": round(prompt_tokens / ms_prefill * 1e3, 1)},
            "decode": {"ms_per_token_step": round(ms_decode / gen, 3), "sequences": n_seqs, "mean_context": round(ctx, 1),
                       "tokens_per_s": round(n_seqs * gen / ms_decode * 1e3, 1)},
            "e2e": {"value": round(n_seqs * gen / ms_decode * 1e3, 1), "unit": "generated tokens/s",
                    "h2d_bytes_per_step": n_seqs * 8, "d2h_bytes_per_step": n_seqs * 8},
            "build_s": round(t_build, 1), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
            "tp_collectives": None if ops is None else dict(ops.calls, nvls=bool(ops.nvls)),
            "reference_arm": "not run: the reference's FastGen (inference v2) needs its CUTLASS / flash-attn extension builds and a 140 GB HF "
                             "checkpoint; its v1 AutoTP path needs the 70B HF module materialised per rank",
        }
        config = {"model": "llama-2-70b" + (f"-{L}layers-INVALID-debug" if args.layers else ""), "parallelism": f"tp{world}",
                  "quantization": args.quant or "bf16", "sequences": n_seqs, "prompt_len": [args.prompt_min, args.prompt_max],
                  "token_budget_per_forward": budget, "generated_tokens_per_timed_step": gen, "kv_block": 128,
                  "l2_policy": "weights (17.5 GB / rank at TP=8) and KV far exceed the 126 MB L2; no explicit flush"}
        print(json.dumps(_line("generated tokens/sec/box Llama-2-70B FastGen ragged decode (TP over all GPUs); prefill tokens/s alongside",
                               n_seqs * gen / ms_decode * 1e3, "tokens/s", world, args, ms_decode, config, clocks, launches, extra)), flush=True)


# ------------------------------------------------------------------------------------------------ config #4: Mixtral EP
def run_mixtral(args):
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.models.mixtral import MixtralForCausalLM, mixtral_config
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {"ep_size": min(world, 8), "activation_checkpointing": True}
    if args.layers:
        over["num_hidden_layers"] = args.layers
    cfg = mixtral_config("8x7b", **over)
    torch.manual_seed(1234 + rank)  # experts differ per rank; the engine broadcasts the shared parameters from rank 0
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = MixtralForCausalLM(cfg)
    torch.set_default_dtype(prev)
    ds = {"train_micro_batch_size_per_gpu": args.micro_batch, "gradient_accumulation_steps": 1, "steps_per_print": 1000000,
          "bf16": {"enabled": True}, "gradient_clipping": 1.0,
          "optimizer": {"type": "AdamW", "params": {"lr": 1e-5, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1}},
          "zero_optimization": {"stage": 2, "overlap_comm": True, "contiguous_gradients": True, "reduce_bucket_size": 5e8}}
    engine, _, _, _ = deepspeed.initialize(model=model, config=ds)
    B, S, V = args.micro_batch, args.seq_len, cfg.vocab_size
    g = torch.Generator().manual_seed(1000 + rank)
    host_ids = torch.randint(0, V, (B, S), generator=g).pin_memory()
    host_labels = torch.randint(0, V, (B, S), generator=g).pin_memory()
    last = {}

    def step():
        ids, labels = host_ids.to(dev, non_blocking=True), host_labels.to(dev, non_blocking=True)
        loss = engine(ids, labels)
        engine.backward(loss)
        engine.step()
        last["loss"] = loss.item()

    l0 = native.launch_count
    ms, clocks = _timed(torch, dist, step, args.steps, args.warmup)
    launches = native.launch_count - l0
    if rank == 0:
        from deepspeedsyclsupport_b200.moe import sharded_moe as SM
        tokens = world * B * S
        n_params = sum(p.numel() for p in model.parameters())
        extra = {"e2e": {"value": tokens / ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8, "d2h_bytes_per_step": 4},
                 "final_loss": last.get("loss"), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
                 "params_per_rank_b": round(n_params / 1e9, 2),
                 "moe_transport": "peer dispatch-push / combine-pull kernels" if os.environ.get("DSB200_MOE_PEER", "1") != "0" else "nccl all-to-all",
                 "reference_arm": "not run (the reference's MoE + ZeRO-2 on this model needs its fused-kernel JIT builds, which fail for sm_100: see DESIGN.md)"}
        config = {"model": "mixtral-8x7b" + (f"-{args.layers}layers-INVALID-debug" if args.layers else ""), "global_batch": B * world, "seq_len": S,
                  "micro_batch_per_gpu": B, "parallelism": f"ep{min(world, 8)}-zero2-dp{world}", "top_k": 2, "capacity_factor": cfg.capacity_factor,
                  "optimizer": "AdamW", "grad_clip": 1.0, "activation_checkpointing": "full",
                  "l2_policy": "working set far exceeds the 126 MB L2; no explicit flush"}
        line = _line("tokens/sec/box Mixtral-8x7B expert-parallel training step (fwd+bwd+AdamW, ZeRO-2)", tokens / ms * 1e3, "tokens/s", world, args,
                     ms, config, clocks, launches, extra)
        line["scaling"] = "weak"
        print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ config #3: Ulysses 13B
def run_ulysses13b(args):
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.models import LlamaForCausalLM, llama_config
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    over = {"activation_checkpointing": True}
    if args.layers:
        over["num_hidden_layers"] = args.layers
    cfg = llama_config("13b", **over)
    assert cfg.num_attention_heads % world == 0, f"{cfg.num_attention_heads} heads do not split over {world} ranks"
    torch.manual_seed(1234)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg)
    torch.set_default_dtype(prev)
    model.set_sequence_parallel(dist.get_world_group())
    ds = {"train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 1, "steps_per_print": 1000000, "bf16": {"enabled": True},
          "gradient_clipping": 1.0,
          "optimizer": {"type": "AdamW", "params": {"lr": 1e-5, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1}},
          "zero_optimization": {"stage": 3, "overlap_comm": True, "contiguous_gradients": True, "stage3_prefetch_bucket_size": 5e8,
                                "stage3_max_live_parameters": 1e10, "stage3_param_persistence_threshold": 1e5, "reduce_bucket_size": 5e8}}
    engine, _, _, _ = deepspeed.initialize(model=model, config=ds)
    S = args.seq_len
    S_local = S // world
    g = torch.Generator().manual_seed(1000)
    host_ids = torch.randint(0, cfg.vocab_size, (1, S), generator=g)[:, rank * S_local:(rank + 1) * S_local].contiguous().pin_memory()
    host_labels = torch.randint(0, cfg.vocab_size, (1, S), generator=g)[:, rank * S_local:(rank + 1) * S_local].contiguous().pin_memory()
    last = {}

    def step():
        ids, labels = host_ids.to(dev, non_blocking=True), host_labels.to(dev, non_blocking=True)
        loss = engine(ids, labels)
        engine.backward(loss)
        engine.step()
        last["loss"] = loss.item()

    l0 = native.launch_count
    ms, clocks = _timed(torch, dist, step, args.steps, args.warmup)
    launches = native.launch_count - l0
    if rank == 0:
        from deepspeedsyclsupport_b200.sequence import fused as UF
        flops_tok = model.flops_per_token(S, with_recompute=False)
        extra = {"e2e": {"value": S / ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 2 * S_local * 8, "d2h_bytes_per_step": 4},
                 "final_loss": last.get("loss"), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
                 "model_flops_per_token": flops_tok, "tflops_per_gpu": round(S / ms * 1e3 * flops_tok / world / 1e12, 1),
                 "ulysses_transport": "peer heads-exchange kernels" if UF._Exchange._by_group else "nccl all-to-all",
                 "reference_arm": "not run (HF Llama + reference DistributedAttention at 128K needs flash-attn inside the reference stack)"}
        config = {"model": "llama-2-13b" + (f"-{args.layers}layers-INVALID-debug" if args.layers else ""), "global_batch": 1, "seq_len": S,
                  "parallelism": f"ulysses-sp{world}-zero3", "heads_per_rank": cfg.num_attention_heads // world, "optimizer": "AdamW",
                  "grad_clip": 1.0, "activation_checkpointing": getattr(model.model, "_policy_cache", (None, "auto"))[1],
                  "l2_policy": "working set far exceeds the 126 MB L2; no explicit flush"}
        print(json.dumps(_line("tokens/sec/box Llama-2-13B Ulysses sequence-parallel ZeRO-3 training step at long context", S / ms * 1e3, "tokens/s",
                               world, args, ms, config, clocks, launches, extra)), flush=True)



# ------------------------------------------------------------------------------------------------ Linasun beside Mixtral (FastGen, 1 GPU)
LINASUN_SIZES = {
    # name: (width, layers, heads, head dim, kv heads of the Mixtral twin, latent rank, query rank, experts, top, ff, vocab)
    "s": (2048, 4, 16, 128, 4, 128, 512, 8, 2, 1024, 32000),
    "m": (4096, 4, 32, 128, 8, 128, 1024, 8, 2, 2048, 32000),
    "l": (6144, 2, 48, 128, 8, 128, 1536, 16, 4, 2048, 32000),
}


def _linasun_state(torch, dev, W, L, H, d, R, Q, E, top, ff, V):
    cfg = {"architecture": "Linasun", "vocab": V, "width": W, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "loop": {"start": 0, "stop": 0, "times": 1},
           "layers": [{"type": "latent_attention", "mixer": {"heads": H, "dim": d, "vdim": d, "kv_rank": R, "q_rank": Q, "scale": d ** -0.5},
                       "mlp": {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": E, "top": top, "groups": {"count": 4, "keep": 2}}}}
                      for _ in range(L)]}

    def r(*shape, std=0.02):
        return torch.empty(*shape, device=dev, dtype=torch.bfloat16).normal_(0.0, std)

    sd = {"embed": r(V, W, std=1.0), "final.norm": r(W), "head": r(V, W)}
    for i in range(L):
        p = f"l{i}."
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            sd[p + n] = r(W)
        sd.update({p + "mix.dq": r(Q, W), p + "mix.dq.norm": r(Q) + 1, p + "mix.uq": r(H * d, Q), p + "mix.dkv": r(R, W), p + "mix.dkv.norm": r(R) + 1,
                   p + "mix.uk": r(H * d, R), p + "mix.uv": r(H * d, R), p + "mix.g": r(H * d, W), p + "mix.o": r(W, H * d),
                   p + "mlp.router": r(E, W, std=0.5), p + "mlp.correction": r(E)})
        for e in range(E):
            sd.update({p + f"mlp.e{e}.gate": r(ff, W), p + f"mlp.e{e}.up": r(ff, W), p + f"mlp.e{e}.down": r(W, ff)})
    return cfg, sd


def _mixtral_state(torch, dev, W, L, H, d, hkv, E, top, ff, V):
    cfg = dict(vocab_size=V, hidden_size=W, intermediate_size=ff, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=hkv,
               rms_norm_eps=1e-5, rope_theta=1e6, max_position_embeddings=8192, num_local_experts=E, num_experts_per_tok=top)
    assert H * d == W, "the Mixtral twin derives its head size from hidden / heads"

    def r(*shape, std=0.02, one=False):
        t = torch.empty(*shape, device=dev, dtype=torch.bfloat16).normal_(0.0, std)
        return t + 1 if one else t

    sd = {"model.embed_tokens.weight": r(V, W, std=1.0), "model.norm.weight": r(W, one=True), "lm_head.weight": r(V, W)}
    for i in range(L):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": r(H * d, W), p + "self_attn.k_proj.weight": r(hkv * d, W), p + "self_attn.v_proj.weight": r(hkv * d, W),
                   p + "self_attn.o_proj.weight": r(W, H * d), p + "block_sparse_moe.gate.weight": r(E, W, std=0.5),
                   p + "input_layernorm.weight": r(W, one=True), p + "post_attention_layernorm.weight": r(W, one=True)})
        for e in range(E):
            sd.update({p + f"block_sparse_moe.experts.{e}.w1.weight": r(ff, W), p + f"block_sparse_moe.experts.{e}.w3.weight": r(ff, W),
                       p + f"block_sparse_moe.experts.{e}.w2.weight": r(W, ff)})
    return cfg, sd


def _event_ms(torch, fn, iters, flush):
    """Median device time of fn() over `iters` runs, an L2 flush (a 256 MB write) before every run, 3 warm-up runs."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.fill_(1.0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def _linasun_kernel_table(torch, peaks, W, H, d, hkv, R, E, top, ff, T, ctx, n_dec):
    """Every kernel of the new design beside the like kernel of the Mixtral path, isolated, with the fraction of the measured roofline
    (HBM copy bandwidth for the streaming kernels, cuBLAS bf16 rate for attention prefill)."""
    from deepspeedsyclsupport_b200.inference.v2 import kernels as K
    from deepspeedsyclsupport_b200.ops import fused_ops as FO
    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, ms, like, like_ms, nbytes=None, like_bytes=None, flops=None, like_flops=None):
        def frac(ms_, b, f):
            return round(max((b or 0) / hbm, (f or 0) / tf) / (ms_ * 1e-3), 3)
        rows.append({"kernel": name, "ms": round(ms, 4), "roofline_frac": frac(ms, nbytes, flops), "like": like, "like_ms": round(like_ms, 4),
                     "like_roofline_frac": frac(like_ms, like_bytes if like_bytes is not None else nbytes, like_flops if like_flops is not None else flops)})

    # norms: fused (branch norm + add + next norm) on an fp32 stream vs fused (add + norm) on a bf16 stream
    x32, y, g32 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf), torch.randn(W, device=dev)
    xb, gb = torch.randn(T, W, device=dev).to(bf), torch.randn(W, device=dev).to(bf)
    add("sandwich_norm (fp32 stream)", _event_ms(torch, lambda: K.sandwich_norm(x32, y, g32, 1.0, g32, 1.0, 1e-6), 20, flush),
        "rms_norm + residual add (bf16 stream)", _event_ms(torch, lambda: FO.rms_norm(y, gb, 1e-5, xb), 20, flush),
        nbytes=T * W * (4 + 4 + 2 + 2), like_bytes=T * W * (2 + 2 + 2 + 2))
    # routers
    lg = torch.randn(T, E, device=dev)
    corr = torch.randn(E, device=dev)
    add("grouped_topk_gating", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top, corr, 4, 2), 20, flush),
        "top_k_gating", _event_ms(torch, lambda: K.top_k_gating(lg, top), 20, flush), nbytes=T * (E * 4 + top * 12))
    counts, scores, asg, off = K.top_k_gating(lg, top)
    h = torch.randn(T, W, device=dev).to(bf)
    add("moe_scatter_rows", _event_ms(torch, lambda: K.moe_scatter_rows(h, counts, asg, off), 20, flush),
        "moe_scatter", _event_ms(torch, lambda: K.moe_scatter(h, counts, asg, off), 20, flush), nbytes=T * W * 2 * (1 + top))
    moe_in, cumsum, slots = K.moe_scatter(h, counts, asg, off)
    dn = torch.randn(T * top, W, device=dev).to(bf)
    add("moe_gather_rows (fp32 out)", _event_ms(torch, lambda: K.moe_gather_rows(dn, scores, slots), 20, flush),
        "moe_gather (bf16 out)", _event_ms(torch, lambda: K.moe_gather(dn, scores, slots), 20, flush),
        nbytes=T * W * (2 * top + 4), like_bytes=T * W * (2 * top + 2))
    gu = torch.randn(T * top, 2 * ff, device=dev).to(bf)
    add("clamped_swish_gate", _event_ms(torch, lambda: K.clamped_swish_gate(gu, 1.702, 7.0, 1.0), 20, flush),
        "gated_act (silu)", _event_ms(torch, lambda: FO.gated_act(gu, "silu"), 20, flush), nbytes=T * top * ff * 6)
    # attention: one prompt portion of T tokens after ctx cached tokens; then n_dec decode tokens at context ctx
    bs = 128
    for label, n_seq, new, seen in (("prefill", max(1, T // 2048), min(T, 2048), ctx), ("decode", n_dec, 1, ctx), ("decode 16K", n_dec, 1, 8 * ctx)):
        per = -(-(seen + new) // bs)
        nb = n_seq * per
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(n_seq, per)
        tok_seq = torch.arange(n_seq, dtype=torch.int32, device=dev).repeat_interleave(new)
        tok_pos = (seen + torch.arange(new, dtype=torch.int32, device=dev)).repeat(n_seq)
        Tn = n_seq * new
        lat_cache = torch.randn(nb, bs, R, device=dev).to(bf)
        Hp = 1 << (H - 1).bit_length()  # the module pads the query heads to a divisor of 128 (useful FLOPs below count H)
        qa = torch.randn(Tn, Hp, R, device=dev).to(bf)
        kv = torch.randn(nb, 2, bs, hkv, d, device=dev).to(bf)
        qkv = torch.randn(Tn, (H + 2 * hkv) * d, device=dev).to(bf)
        dec = label.startswith("decode")
        keys = n_seq * (new * seen + new * (new + 1) // 2)  # (query, key) pairs
        fl_lat, fl_std = 4.0 * keys * H * R, 4.0 * keys * H * d
        by_lat, by_std = nb * bs * R * 2 + Tn * H * R * 4, nb * bs * hkv * d * 4 + Tn * H * d * 4
        add(f"latent attention, {label} (tcgen05, one plane)", _event_ms(torch, lambda: K.paged_latent_flash(qa, lat_cache, tok_seq, tok_pos, bt, d ** -0.5, decode=dec), 10, flush),
            f"paged flash attention, {label} (GQA {H}:{hkv})", _event_ms(torch, lambda: K.paged_attention(qkv, kv, tok_seq, tok_pos, bt, H, hkv, d, d ** -0.5, decode=dec), 10, flush),
            nbytes=by_lat, like_bytes=by_std, flops=fl_lat, like_flops=fl_std)
        if dec:
            qf = qa[:, :H].float()
            add("latent attention, decode (CUDA cores, fp32)", _event_ms(torch, lambda: K.latent_attention(qf, lat_cache, tok_seq, tok_pos, bt, d ** -0.5, max_keys=seen + 1), 5, flush),
                f"paged flash attention, decode (GQA {H}:{hkv})", rows[-1]["like_ms"], nbytes=by_lat, like_bytes=by_std, flops=0, like_flops=0)
    return rows


def run_linasun(args):
    """Prefill and decode throughput of Linasun through the FastGen engine at a few layer sizes, beside a Mixtral of equal size
    (same width, layers, heads, experts, ff, top-k, vocabulary), plus the isolated kernels of the new design beside their likes."""
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.inference.v2 import RaggedInferenceEngineConfig, build_engine_from_state_dict
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    assert dist.get_world_size() == 1, "--workload linasun is a one-GPU comparison"
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        peaks = dict(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), source="measured")
    n_seqs, prompt, budget = min(args.sequences, 64), 1024, 4096
    results, clocks, l0 = {}, None, native.launch_count
    g = torch.Generator().manual_seed(11)
    for name in (args.model.split(",") if args.model != "7b" else ["s", "m", "l"]):
        W, L, H, d, hkv, R, Q, E, top, ff, V = LINASUN_SIZES[name]
        max_ctx = -(-(prompt + 4 * (args.steps + args.warmup) * 4 + 64) // 128) * 128
        ecfg = RaggedInferenceEngineConfig(state_manager={"max_ragged_batch_size": budget, "max_ragged_sequence_count": n_seqs, "max_tracked_sequences": n_seqs,
                                                          "max_context": max_ctx, "memory_config": {"mode": "allocate", "size": n_seqs * (max_ctx // 128) + 4}})
        res = {}
        for fam in ("linasun", "mixtral"):
            cfg, sd = _linasun_state(torch, dev, W, L, H, d, R, Q, E, top, ff, V) if fam == "linasun" else _mixtral_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            eng = build_engine_from_state_dict(fam, cfg, sd, ecfg, dtype=torch.bfloat16)
            n_params = sum(v.numel() for v in sd.values())
            del sd
            prompts = [torch.randint(0, V, (prompt, ), generator=g).pin_memory() for _ in range(n_seqs)]
            uids = list(range(n_seqs))
            state = {"live": False, "next": None}

            def prefill():
                if state["live"]:
                    for u in uids:
                        eng.flush(u)
                per = budget // prompt
                nxt = torch.zeros(n_seqs, dtype=torch.long)
                for i in range(0, n_seqs, per):
                    us = uids[i:i + per]
                    nxt[i:i + len(us)] = eng.put(us, [prompts[u] for u in us]).argmax(-1).cpu()
                state["live"], state["next"] = True, nxt

            def decode():
                nxt = state["next"]
                for _ in range(4):
                    nxt = eng.put(uids, [nxt[u:u + 1] for u in uids]).argmax(-1).cpu()
                state["next"] = nxt

            ms_p, _ = _timed(torch, dist, prefill, args.steps, 3)
            ms_d, clocks = _timed(torch, dist, decode, args.steps, args.warmup)
            res[fam] = {"params_b": round(n_params / 1e9, 3), "prefill_tokens_per_s": round(n_seqs * prompt / ms_p * 1e3, 1), "prefill_ms": round(ms_p, 2),
                        "decode_tokens_per_s": round(n_seqs * 4 / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d / 4, 3)}
            del eng
            torch.cuda.empty_cache()
        res["linasun_over_mixtral"] = {"prefill": round(res["linasun"]["prefill_tokens_per_s"] / res["mixtral"]["prefill_tokens_per_s"], 3),
                                       "decode": round(res["linasun"]["decode_tokens_per_s"] / res["mixtral"]["decode_tokens_per_s"], 3)}
        res["shape"] = {"width": W, "layers": L, "heads": H, "head_dim": d, "mixtral_kv_heads": hkv, "kv_rank": R, "q_rank": Q, "experts": E, "top": top, "ff": ff}
        res["kernels"] = _linasun_kernel_table(torch, peaks, W, H, d, hkv, R, E, top, ff, 4096, 2048, n_seqs)
        results[name] = res
    launches = native.launch_count - l0
    last = results[list(results)[-1]]
    extra = {"results": results, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
             "e2e": {"value": last["linasun"]["decode_tokens_per_s"], "unit": "generated tokens/s", "h2d_bytes_per_step": n_seqs * 8, "d2h_bytes_per_step": n_seqs * 8},
             "reference_arm": "none: the reference has no model of this design"}
    config = {"model": "linasun (random weights) beside mixtral of equal size", "sizes": list(results), "sequences": n_seqs, "prompt_len": prompt,
              "token_budget_per_forward": budget, "decode_steps_per_timed_step": 4, "kv_block": 128,
              "l2_policy": "engine steps: weights exceed the 126 MB L2, no flush; isolated kernels: 256 MB write before every timed run"}
    print(json.dumps(_line("generated tokens/sec Linasun FastGen ragged decode, 1 GPU (prefill and a Mixtral of equal size alongside)",
                           last["linasun"]["decode_tokens_per_s"], "tokens/s", 1, args, last["linasun"]["decode_ms_per_step"], config, clocks, launches, extra)),
          flush=True)


# ---- Kulanex beside a Mixtral of equal size
KULANEX_SIZES = {  # width, layers, attention heads, head_dim, kv heads, window, experts, top, ff, vocab
    "s": (2048, 4, 16, 128, 4, 1024, 8, 2, 1024, 32000),
    "m": (4096, 4, 32, 128, 8, 1024, 8, 2, 2048, 32000),
}


def _kulanex_state(torch, dev, W, L, H, d, hkv, window, E, top, ff, V):
    """Layers alternate 'parallel' (windowed attention H:hkv x d beside a matrix memory of H/2 heads, 64 x 2d) and 'channel_delta'
    (H heads, d x d), all with the MoE feed-forward; the layer input projections add up to about the twin's."""
    mh, md, mv, lr = H // 2, 64, 2 * d, 128
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    par = {"type": "parallel", "mlp": moe,
           "mixer": {"left": {"conv": 4, "dim": d, "heads": H, "kv_heads": hkv, "mask": {"keep_first": 4, "size": window},
                              "rot": {"base": 1e6, "dims": d // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}, "scale": d ** -0.5, "vdim": d},
                     "left_scale": 1.0, "right": {"dim": md, "gate_cap": 15.0, "heads": mh, "vdim": mv}, "right_scale": 1.0}}
    dl = {"type": "channel_delta", "mlp": moe, "mixer": {"conv": 4, "dim": d, "heads": H, "kv_heads": H, "vdim": d}}
    cfg = {"architecture": "Kulanex", "vocab": V, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": [par if i % 2 == 0 else dl for i in range(L)]}

    def r(*shape, std=0.02, mean=0.0):
        return torch.empty(*shape, device=dev, dtype=torch.bfloat16).normal_(mean, std)

    sd = {"embed": r(V, W, std=1.0), "final.norm": r(W), "head": r(V, W)}
    for i in range(L):
        p = f"l{i}."
        sd.update({p + "norm1": r(W), p + "norm2": r(W), p + "mlp.router": r(E, W, std=0.5)})
        for e in range(E):
            sd.update({p + f"mlp.e{e}.gate": r(ff, W), p + f"mlp.e{e}.up": r(ff, W), p + f"mlp.e{e}.down": r(W, ff)})
        if i % 2 == 0:
            a, b = p + "mix.left.", p + "mix.right."
            sd.update({a + "q": r(H * d, W), a + "k": r(hkv * d, W), a + "q.conv": r(H * d, 4, std=0.5), a + "k.conv": r(hkv * d, 4, std=0.5),
                       a + "q.norm": r(H * d, mean=1.0), a + "k.norm": r(hkv * d, mean=1.0), a + "o": r(W, H * d),
                       b + "q": r(mh * md, W), b + "k": r(mh * md, W), b + "v": r(mh * mv, W), b + "g": r(mh * mv, W), b + "o": r(W, mh * mv),
                       b + "norm": r(mh * mv, mean=1.0), b + "i": r(mh, W), b + "i.b": r(mh), b + "f": r(mh, W), b + "f.b": r(mh, mean=3.0)})
        else:
            a = p + "mix."
            sd.update({a + "q": r(H * d, W), a + "k": r(H * d, W), a + "v": r(H * d, W), a + "q.conv": r(H * d, 4, std=0.5), a + "k.conv": r(H * d, 4, std=0.5),
                       a + "v.conv": r(H * d, 4, std=0.5), a + "b": r(H, W), a + "A_log": r(H, mean=-2.5), a + "norm": r(d, mean=1.0), a + "a1": r(lr, W),
                       a + "a2": r(H * d, lr), a + "dt_bias": r(H * d, mean=-2.0), a + "g1": r(lr, W), a + "g2": r(H * d, lr), a + "o": r(W, H * d)})
    return cfg, sd


def _kulanex_kernel_table(torch, peaks, W, H, d, hkv, window, E, top, ff, T, ctx, n_dec):
    """Every kernel of the design beside the like kernel of the Mixtral path, isolated, with the fraction of the measured roofline (HBM copy
    bandwidth for the streaming kernels, cuBLAS bf16 rate for attention prefill).  The recurrent scans have no like among the attention
    models' kernels but the attention itself; they are listed beside it with their own bytes (inputs + outputs + the state once in, once out)."""
    from deepspeedsyclsupport_b200.inference.v2 import kernels as K
    from deepspeedsyclsupport_b200.ops import fused_ops as FO
    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, ms, like, like_ms, nbytes=None, like_bytes=None, flops=None, like_flops=None):
        def frac(ms_, b, f):
            return round(max((b or 0) / hbm, (f or 0) / tf) / (ms_ * 1e-3), 3)
        rows.append({"kernel": name, "ms": round(ms, 4), "roofline_frac": frac(ms, nbytes, flops), "like": like, "like_ms": round(like_ms, 4),
                     "like_roofline_frac": frac(like_ms, like_bytes if like_bytes is not None else nbytes, like_flops if like_flops is not None else flops)})

    x32, y, g32 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf), torch.randn(W, device=dev)
    xb, gb = torch.randn(T, W, device=dev).to(bf), torch.randn(W, device=dev).to(bf)
    add("post-norm into the fp32 stream + bf16 copy", _event_ms(torch, lambda: K.sandwich_norm(x32, y, g32, 1.0, None, 0.0, 1e-6, y_mult=0.5, plain_out=True), 20, flush),
        "rms_norm + residual add (bf16 stream)", _event_ms(torch, lambda: FO.rms_norm(y, gb, 1e-5, xb), 20, flush),
        nbytes=T * W * (4 + 4 + 2 + 2), like_bytes=T * W * (2 + 2 + 2 + 2))
    lg = torch.randn(T, E, device=dev)
    add("grouped_topk_gating (sigmoid scores)", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top, sigmoid_scores=True), 20, flush),
        "top_k_gating", _event_ms(torch, lambda: K.top_k_gating(lg, top), 20, flush), nbytes=T * (E * 4 + top * 12))
    counts, scores, asg, off = K.top_k_gating(lg, top)
    h = torch.randn(T, W, device=dev).to(bf)
    add("moe_scatter_rows (scaled copies)", _event_ms(torch, lambda: K.moe_scatter_rows(h, counts, asg, off, row_scale=scores), 20, flush),
        "moe_scatter", _event_ms(torch, lambda: K.moe_scatter(h, counts, asg, off), 20, flush), nbytes=T * W * 2 * (1 + top))
    moe_in, cumsum, slots = K.moe_scatter(h, counts, asg, off)
    dn = torch.randn(T * top, W, device=dev).to(bf)
    add("moe_gather_rows (plain sum, fp32 out)", _event_ms(torch, lambda: K.moe_gather_rows(dn, None, slots), 20, flush),
        "moe_gather (bf16 out)", _event_ms(torch, lambda: K.moe_gather(dn, scores, slots), 20, flush),
        nbytes=T * W * (2 * top + 4), like_bytes=T * W * (2 * top + 2))
    # token mixers: one prompt portion per sequence after ctx cached tokens; then n_dec decode tokens at context ctx
    bs = 128
    mh, md, mv = H // 2, 64, 2 * d
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import scaled_rotary_frequencies
    freq = scaled_rotary_frequencies(d // 2, 1e6, None).to(dev)
    inv_freq = (1e6 ** (-torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))
    for label, n_seq, new, seen in (("prefill", max(1, T // 2048), min(T, 2048), ctx), ("decode", n_dec, 1, ctx)):
        per = -(-(seen + new) // bs)
        nb = n_seq * per
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(n_seq, per)
        tok_seq = torch.arange(n_seq, dtype=torch.int32, device=dev).repeat_interleave(new)
        tok_pos = (seen + torch.arange(new, dtype=torch.int32, device=dev)).repeat(n_seq)
        desc = torch.tensor([[i * new, new, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        Tn = n_seq * new
        dec = label == "decode"
        kv = torch.randn(nb, 2, bs, hkv, d, device=dev).to(bf)
        qkv = torch.randn(Tn, (H + 2 * hkv) * d, device=dev).to(bf)
        # q / k preparation (convolution, norms, rotation, append) vs rotary + append
        C = (H + hkv) * d
        proj = torch.randn(Tn, C, device=dev).to(bf)
        cw, nw = torch.randn(C, 4, device=dev), torch.randn(C, device=dev)
        cstate = torch.zeros(n_seq, 3, C, device=dev, dtype=bf)
        qo = torch.empty(Tn, H * d, device=dev, dtype=bf)

        def prep():
            K.window_qk_prepare(proj, 0, H * d, cw, cw[H * d:], nw, nw[H * d:], cstate, desc, tok_seq, tok_pos, bt, kv, qo, freq, H, hkv, d, 4, d // 2, 1e-6)
            K.conv_state_update(proj, 0, C, cstate, 0, desc, n_seq, 4)
        add(f"window_qk_prepare + conv_state_update, {label}", _event_ms(torch, prep, 10, flush),
            f"kv_rotary_append, {label}", _event_ms(torch, lambda: K.kv_rotary_append(qkv, kv, tok_seq, tok_pos, bt, inv_freq, H, hkv, d), 10, flush),
            nbytes=Tn * (C * 2 + H * d * 2 + 2 * hkv * d * 2), like_bytes=Tn * ((H + 2 * hkv) * d * 2 * 2 - H * d * 0 + 0))
        vis = min(window, seen + new)  # keys a query sees (about)
        keys = n_seq * new * vis
        out = torch.empty(Tn, H * d, device=dev, dtype=bf)
        from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import windowed_attention
        add(f"windowed attention with kept tokens, {label}", _event_ms(torch, lambda: windowed_attention(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, window, 4, d ** -0.5, 1.0, decode=dec), 10, flush),
            f"paged flash attention, window {window}, {label} (GQA {H}:{hkv})",
            _event_ms(torch, lambda: K.paged_attention(qkv, kv, tok_seq, tok_pos, bt, H, hkv, d, d ** -0.5, decode=dec, window=window), 10, flush),
            nbytes=n_seq * min(seen + new, window + new) * hkv * d * 4 + Tn * H * d * 4, flops=4.0 * keys * H * d)
        # recurrent scans
        like_ms, like_frac_b = rows[-1]["like_ms"], n_seq * min(seen + new, window + new) * hkv * d * 4 + Tn * H * d * 4
        pm = torch.randn(Tn, mh * (2 * md + 2 * mv), device=dev).to(bf) * 0.1
        gates = torch.randn(Tn, 2 * mh, device=dev)
        bi, bfg = torch.zeros(mh, device=dev), torch.full((mh, ), 3.0, device=dev)
        sS = torch.zeros(n_seq, mh, K.scan_state_floats(md, mv), device=dev)
        sn, smx = torch.zeros(n_seq, mh, md, device=dev), torch.zeros(n_seq, mh, device=dev)
        state_b = n_seq * mh * md * mv * 4 * 2
        add(f"matrix_memory_scan ({mh} x {md} x {mv}), {label}",
            _event_ms(torch, lambda: K.matrix_memory_scan(pm, 0, mh * md, 2 * mh * md, gates, bi, bfg, 15.0, desc, n_seq, sS, sn, smx, mh, md, mv), 5, flush),
            f"paged flash attention, {label}", like_ms, nbytes=Tn * mh * (2 * md + mv) * 2 + Tn * mh * mv * 4 + state_b, like_bytes=like_frac_b,
            flops=0, like_flops=4.0 * keys * H * d)
        qn, kn, vv = torch.randn(Tn, H * d, device=dev) * 0.1, torch.randn(Tn, H * d, device=dev) * 0.1, torch.randn(Tn, H * d, device=dev)
        bp, ap = torch.randn(Tn, H, device=dev), torch.randn(Tn, H * d, device=dev)
        Al, dtb = torch.full((H, ), -2.5, device=dev), torch.full((H * d, ), -2.0, device=dev)
        dS = torch.zeros(n_seq, H, K.scan_state_floats(d, d), device=dev)
        bp, ap = torch.sigmoid(bp), torch.exp(-0.08 * torch.nn.functional.softplus(ap - 2.0))  # betas and decays as delta_prepare leaves them
        add(f"delta_rule_scan ({H} x {d} x {d}), {label}", _event_ms(torch, lambda: K.delta_rule_scan(qn, kn, vv, bp, ap, desc, n_seq, dS, H, H, d, d), 5, flush),
            f"paged flash attention, {label}", like_ms, nbytes=Tn * H * (4 * d * 4 + 4) + Tn * H * d * 4 + n_seq * H * d * d * 8, like_bytes=like_frac_b,
            flops=0, like_flops=4.0 * keys * H * d)
        p3 = torch.randn(Tn, 3 * H * d, device=dev).to(bf)
        c3 = torch.randn(3 * H * d, 4, device=dev)
        st3 = torch.zeros(n_seq, 3, 3 * H * d, device=dev, dtype=bf)
        ap2, bp2 = torch.randn(Tn, H * d, device=dev), torch.randn(Tn, H, device=dev)

        def dprep():
            K.delta_prepare(p3, 0, H * d, 2 * H * d, c3, c3[H * d:], c3[2 * H * d:], st3, desc, tok_seq, ap2, bp2, Al, dtb, H, H, d, d, 4)
            K.conv_state_update(p3, 0, 3 * H * d, st3, 0, desc, n_seq, 4)
        add(f"delta_prepare + conv_state_update, {label}", _event_ms(torch, dprep, 10, flush), f"kv_rotary_append, {label}", rows[-4]["like_ms"],
            nbytes=Tn * (3 * H * d * (2 + 4) + H * d * 8), like_bytes=Tn * (H + 2 * hkv) * d * 4)
        o32, gt, og = torch.randn(Tn, H * d, device=dev), torch.randn(Tn, H * d, device=dev).to(bf), torch.empty(Tn, H * d, device=dev, dtype=bf)
        add(f"head_norm_gate, {label}", _event_ms(torch, lambda: K.head_norm_gate(o32, nw[:d].contiguous(), gt, og, H, d, 1e-6, shared_weight=True), 10, flush),
            "gated_act (silu)", _event_ms(torch, lambda: FO.gated_act(torch.cat([gt, gt], 1) if False else qkv[:, :2 * (H * d // 2)].contiguous(), "silu"), 10, flush),
            nbytes=Tn * H * d * 8, like_bytes=Tn * H * d * 3)
    return rows


def run_kulanex(args):
    """Prefill and decode throughput of Kulanex through the FastGen engine at a few layer sizes, beside a Mixtral of equal size (same
    width, layers, heads, experts, ff, top-k, vocabulary), plus the isolated kernels of the design beside their likes."""
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.inference.v2 import RaggedInferenceEngineConfig, build_engine_from_state_dict
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    assert dist.get_world_size() == 1, "--workload kulanex is a one-GPU comparison"
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        peaks = dict(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), source="measured")
    n_seqs, prompt, budget = min(args.sequences, 64), 1024, 4096
    results, clocks, l0 = {}, None, native.launch_count
    g = torch.Generator().manual_seed(11)
    for name in (args.model.split(",") if args.model != "7b" else ["s", "m"]):
        W, L, H, d, hkv, window, E, top, ff, V = KULANEX_SIZES[name]
        max_ctx = -(-(prompt + 4 * (args.steps + args.warmup) * 4 + 64) // 128) * 128
        ecfg = RaggedInferenceEngineConfig(state_manager={"max_ragged_batch_size": budget, "max_ragged_sequence_count": n_seqs, "max_tracked_sequences": n_seqs,
                                                          "max_context": max_ctx, "memory_config": {"mode": "allocate", "size": n_seqs * (max_ctx // 128) + 4}})
        res = {}
        for fam in ("kulanex", "mixtral"):
            cfg, sd = _kulanex_state(torch, dev, W, L, H, d, hkv, window, E, top, ff, V) if fam == "kulanex" else _mixtral_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            eng = build_engine_from_state_dict(fam, cfg, sd, ecfg, dtype=torch.bfloat16)
            n_params = sum(v.numel() for v in sd.values())
            del sd
            prompts = [torch.randint(0, V, (prompt, ), generator=g).pin_memory() for _ in range(n_seqs)]
            uids = list(range(n_seqs))
            state = {"live": False, "next": None}

            def prefill():
                if state["live"]:
                    for u in uids:
                        eng.flush(u)
                per = budget // prompt
                nxt = torch.zeros(n_seqs, dtype=torch.long)
                for i in range(0, n_seqs, per):
                    us = uids[i:i + per]
                    nxt[i:i + len(us)] = eng.put(us, [prompts[u] for u in us]).argmax(-1).cpu()
                state["live"], state["next"] = True, nxt

            def decode():
                nxt = state["next"]
                for _ in range(4):
                    nxt = eng.put(uids, [nxt[u:u + 1] for u in uids]).argmax(-1).cpu()
                state["next"] = nxt

            ms_p, _ = _timed(torch, dist, prefill, args.steps, 3)
            ms_d, clocks = _timed(torch, dist, decode, args.steps, args.warmup)
            res[fam] = {"params_b": round(n_params / 1e9, 3), "prefill_tokens_per_s": round(n_seqs * prompt / ms_p * 1e3, 1), "prefill_ms": round(ms_p, 2),
                        "decode_tokens_per_s": round(n_seqs * 4 / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d / 4, 3)}
            del eng
            torch.cuda.empty_cache()
        res["kulanex_over_mixtral"] = {"prefill": round(res["kulanex"]["prefill_tokens_per_s"] / res["mixtral"]["prefill_tokens_per_s"], 3),
                                       "decode": round(res["kulanex"]["decode_tokens_per_s"] / res["mixtral"]["decode_tokens_per_s"], 3)}
        res["shape"] = {"width": W, "layers": L, "heads": H, "head_dim": d, "kv_heads": hkv, "window": window, "experts": E, "top": top, "ff": ff}
        res["kernels"] = _kulanex_kernel_table(torch, peaks, W, H, d, hkv, window, E, top, ff, 4096, 2048, n_seqs)
        results[name] = res
    launches = native.launch_count - l0
    last = results[list(results)[-1]]
    extra = {"results": results, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
             "e2e": {"value": last["kulanex"]["decode_tokens_per_s"], "unit": "generated tokens/s", "h2d_bytes_per_step": n_seqs * 8, "d2h_bytes_per_step": n_seqs * 8},
             "reference_arm": "none: the reference has no model of this design"}
    config = {"model": "kulanex (random weights) beside mixtral of equal size", "sizes": list(results), "sequences": n_seqs, "prompt_len": prompt,
              "token_budget_per_forward": budget, "decode_steps_per_timed_step": 4, "kv_block": 128,
              "l2_policy": "engine steps: weights exceed the 126 MB L2, no flush; isolated kernels: 256 MB write before every timed run"}
    print(json.dumps(_line("generated tokens/sec Kulanex FastGen ragged decode, 1 GPU (prefill and a Mixtral of equal size alongside)",
                           last["kulanex"]["decode_tokens_per_s"], "tokens/s", 1, args, last["kulanex"]["decode_ms_per_step"], config, clocks, launches, extra)),
          flush=True)


# ---- Pudinex beside a Kulanex and a Mixtral of equal size
PUDINEX_SIZES = {  # width, layers, attention heads, head_dim, kv heads, experts, top, ff, vocab
    "s": (2048, 4, 16, 128, 4, 8, 2, 1024, 32000),
    "m": (4096, 4, 32, 128, 8, 8, 2, 2048, 32000),
}
PUDINEX_IDENTITY = 2


def _pudinex_state(torch, dev, W, L, H, d, hkv, E, top, ff, V):
    """Layers alternate 'hgrn2' (H heads, d x d states) and 'attention' (H:hkv heads of d, half of every head rotated, soft cap 50), all with
    the MoE feed-forward (E experts + 2 identity experts, a shared expert of the experts' size); two norm parts."""
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "identity": PUDINEX_IDENTITY, "top": top}, "shared": {"ff": ff}}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": H, "kv_heads": hkv, "dim": d, "vdim": d, "scale": d ** -0.5, "softcap": 50.0,
                     "rot": {"base": 1e6, "dims": d // 2, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}}
    rec = {"type": "hgrn2", "mlp": moe, "mixer": {"heads": H, "dim": d, "vdim": d}}
    cfg = {"architecture": "Pudinex", "vocab": V, "width": W, "norm": {"eps": 1e-6, "groups": 2}, "embedding": {"scale": 1.0},
           "layers": [rec if i % 2 == 0 else att for i in range(L)]}

    def r(*shape, std=0.02, mean=0.0):
        return torch.empty(*shape, device=dev, dtype=torch.bfloat16).normal_(mean, std)

    sd = {"embed": r(V, W, std=1.0), "final.norm": r(W, mean=1.0), "head": r(V, W)}
    for i in range(L):
        p = f"l{i}."
        sd.update({p + "norm1": r(W, mean=1.0), p + "mlp.router": r(E + PUDINEX_IDENTITY, W, std=0.5), p + "mlp.correction": r(E + PUDINEX_IDENTITY),
                   p + "mlp.shared.gate": r(ff, W), p + "mlp.shared.up": r(ff, W), p + "mlp.shared.down": r(W, ff)})
        for e in range(E):
            sd.update({p + f"mlp.e{e}.gate": r(ff, W), p + f"mlp.e{e}.up": r(ff, W), p + f"mlp.e{e}.down": r(W, ff)})
        a = p + "mix."
        if i % 2 == 0:
            sd.update({a + "q": r(H * d, W), a + "f": r(H * d, W), a + "f.b": r(H * d, mean=2.0, std=1.0), a + "lower": r(H * d, mean=0.5, std=0.1), a + "v": r(H * d, W),
                       a + "norm": r(d, mean=1.0), a + "o": r(W, H * d)})
        else:
            sd.update({a + "q": r(H * d, W), a + "k": r(hkv * d, W), a + "v": r(hkv * d, W), a + "q.norm": r(d, mean=1.0), a + "k.norm": r(d, mean=1.0), a + "o": r(W, H * d)})
    return cfg, sd


def _pudinex_kernel_table(torch, peaks, W, H, d, hkv, E, top, ff, T, ctx, n_dec):
    """Every kernel of the design beside the like kernel of the closest family (Kulanex; the plain Mixtral path where Kulanex has none),
    isolated, with the fraction of the measured roofline (HBM copy bandwidth for the streaming kernels, cuBLAS bf16 rate for attention
    prefill)."""
    from deepspeedsyclsupport_b200.inference.v2 import kernels as K
    from deepspeedsyclsupport_b200.ops import fused_ops as FO
    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, ms, like, like_ms, nbytes=None, like_bytes=None, flops=None, like_flops=None):
        def frac(ms_, b, f):
            return round(max((b or 0) / hbm, (f or 0) / tf) / (ms_ * 1e-3), 3)
        rows.append({"kernel": name, "ms": round(ms, 4), "roofline_frac": frac(ms, nbytes, flops), "like": like, "like_ms": round(like_ms, 4),
                     "like_roofline_frac": frac(like_ms, like_bytes if like_bytes is not None else nbytes, like_flops if like_flops is not None else flops)})

    x32, y, y32, g32 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev), torch.randn(W, device=dev)
    add("stream_group_norm (2 parts; bf16 + fp32 branch in, bf16 + fp32 copy out)",
        _event_ms(torch, lambda: K.stream_group_norm(x32, (y, ), y32, g32, 2, 1e-6, fp32_copy=True), 20, flush),
        "sandwich_norm post-norm into the fp32 stream + bf16 copy (Kulanex)",
        _event_ms(torch, lambda: K.sandwich_norm(x32, y, g32, 1.0, None, 0.0, 1e-6, y_mult=0.5, plain_out=True), 20, flush),
        nbytes=T * W * (4 + 4 + 2 + 4 + 2 + 4), like_bytes=T * W * (4 + 4 + 2 + 2))
    n_out = E + PUDINEX_IDENTITY
    lg, corr = torch.randn(T, n_out, device=dev), torch.randn(n_out, device=dev) * 0.01
    add("grouped_topk_gating (softmax, correction, renormalised)", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top, corr, normalize=True), 20, flush),
        "grouped_topk_gating (sigmoid scores; Kulanex)", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top, sigmoid_scores=True), 20, flush),
        nbytes=T * (n_out * 4 + top * 12))
    counts, scores, asg, off = K.grouped_topk_gating(lg, top, corr, normalize=True)
    h = torch.randn(T, W, device=dev).to(bf)
    moe_in, cumsum, slots = K.moe_scatter_rows(h, counts, asg, off)
    dn = torch.randn(T * top, W, device=dev).to(bf)
    add("moe_gather_rows (identity experts read the fp32 input)", _event_ms(torch, lambda: K.moe_gather_rows(dn, scores, slots, asg, E, y32), 20, flush),
        "moe_gather_rows (plain sum; Kulanex)", _event_ms(torch, lambda: K.moe_gather_rows(dn, None, slots), 20, flush), nbytes=T * W * (2 * top + 4))
    gu = torch.randn(T, 3 * H * d + 2 * ff, device=dev).to(bf)
    wide = torch.empty(T, H * d + ff, device=dev, dtype=bf)
    gpair = torch.randn(T, 2 * ff, device=dev).to(bf)
    add("clamped_swish_gate_cols (column ranges of the fused projection)", _event_ms(torch, lambda: K.clamped_swish_gate_cols(gu, 3 * H * d, 3 * H * d + ff, ff, wide[:, H * d:], 1.0, float("inf"), 0.0), 20, flush),
        "gated_act (silu; Mixtral)", _event_ms(torch, lambda: FO.gated_act(gpair, "silu"), 20, flush), nbytes=T * ff * 6)
    bs = 128
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import RampRotaryScalingConfig
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.sink_blocked_attention import ramp_scaled_frequencies
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import scaled_rotary_frequencies
    freq, mag = ramp_scaled_frequencies(d // 2, 1e6, RampRotaryScalingConfig(factor=8.0, original=8192, fast=32.0, slow=1.0))
    freq = freq.to(dev)
    wfreq = scaled_rotary_frequencies(d // 2, 1e6, None).to(dev)
    inv_freq = (1e6 ** (-torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))
    for label, n_seq, new, seen in (("prefill", max(1, T // 2048), min(T, 2048), ctx), ("decode", n_dec, 1, ctx)):
        per = -(-(seen + new) // bs)
        nb = n_seq * per
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(n_seq, per)
        tok_seq = torch.arange(n_seq, dtype=torch.int32, device=dev).repeat_interleave(new)
        tok_pos = (seen + torch.arange(new, dtype=torch.int32, device=dev)).repeat(n_seq)
        desc = torch.tensor([[i * new, new, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        Tn = n_seq * new
        dec = label == "decode"
        kv = torch.randn(nb, 2, bs, hkv, d, device=dev).to(bf)
        qkv = torch.randn(Tn, (H + 2 * hkv) * d, device=dev).to(bf)
        nw = torch.randn(d, device=dev)
        qo = torch.empty(Tn, H * d, device=dev, dtype=bf)
        planes = K.cache_planes(kv)
        # per-head norms + rotation + append vs the convolving prepare of Kulanex and the plain rotary append
        C = (H + hkv) * d
        cw, cn = torch.randn(C, 4, device=dev), torch.randn(C, device=dev)
        cstate = torch.zeros(n_seq, 3, C, device=dev, dtype=bf)

        def kprep():
            K.window_qk_prepare(qkv, 0, H * d, cw, cw[H * d:], cn, cn[H * d:], cstate, desc, tok_seq, tok_pos, bt, kv, qo, wfreq, H, hkv, d, 4, d // 2, 1e-6)
            K.conv_state_update(qkv, 0, C, cstate, 0, desc, n_seq, 4)
        ms_prep = _event_ms(torch, lambda: K.head_norm_rotary_append(qkv, 0, H * d, (H + hkv) * d, nw, nw, freq, mag, tok_seq, tok_pos, bt, bs, planes[0], planes[1], qo,
                                                                     H, hkv, d, d, d // 2, 1e-6), 10, flush)
        add(f"head_norm_rotary_append, {label}", ms_prep, f"window_qk_prepare + conv_state_update (Kulanex), {label}", _event_ms(torch, kprep, 10, flush),
            nbytes=Tn * (H + 2 * hkv) * d * 4, like_bytes=Tn * (C * 2 + H * d * 2 + 2 * hkv * d * 2))
        add(f"head_norm_rotary_append, {label} ", ms_prep, f"kv_rotary_append (Mixtral), {label}",
            _event_ms(torch, lambda: K.kv_rotary_append(qkv, kv, tok_seq, tok_pos, bt, inv_freq, H, hkv, d), 10, flush), nbytes=Tn * (H + 2 * hkv) * d * 4)
        keys = n_seq * new * (seen + (new + 1) / 2)
        out = torch.empty(Tn, H * d, device=dev, dtype=bf)
        abytes = n_seq * (seen + new) * hkv * d * 4 + Tn * H * d * 4
        add(f"attention, soft cap 50 + sink, tcgen05, {label} (GQA {H}:{hkv})",
            _event_ms(torch, lambda: K.paged_flash_sink(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, d ** -0.5, 50.0, 1.0, decode=dec), 10, flush),
            f"paged flash attention, causal, {label} (Mixtral)",
            _event_ms(torch, lambda: K.paged_attention(qkv, kv, tok_seq, tok_pos, bt, H, hkv, d, d ** -0.5, decode=dec), 10, flush), nbytes=abytes, flops=4.0 * keys * H * d)
        add(f"attention, sink only (no cap), tcgen05, {label}",
            _event_ms(torch, lambda: K.paged_flash_sink(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, d ** -0.5, 0.0, 1.0, decode=dec), 10, flush),
            f"paged flash attention, causal, {label} (Mixtral)", rows[-1]["like_ms"], nbytes=abytes, flops=4.0 * keys * H * d)
        # the CUDA-core kernel that serves fp32 runs and unequal key / value head sizes (here values half as wide as keys)
        kc, vc = torch.randn(nb, bs, hkv, d, device=dev).to(bf), torch.randn(nb, bs, hkv, d // 2, device=dev).to(bf)
        kp, vp = K.cache_planes(kc, vc)
        oh = torch.empty(Tn, H * d // 2, device=dev, dtype=bf)
        add(f"attention, soft cap 50 + sink, CUDA cores, values {d // 2} wide, {label}",
            _event_ms(torch, lambda: K.sink_attention(qo, kp, vp, tok_seq, tok_pos, bt, bs, oh, H, hkv, d, d // 2, d ** -0.5, 50.0, 1.0), 3, flush),
            f"window_attention, CUDA cores, window covering the context (Kulanex), {label}",
            _event_ms(torch, lambda: K.window_attention(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, 1 << 30, 0, d ** -0.5), 3, flush),
            nbytes=n_seq * (seen + new) * hkv * d * 3 + Tn * H * d * 3, like_bytes=abytes, flops=3.0 * keys * H * d, like_flops=4.0 * keys * H * d)
        # recurrent scan beside Kulanex's delta rule on a state of the same size
        proj = torch.randn(Tn, 3 * H * d, device=dev).to(bf)
        fb, lo = torch.full((H * d, ), 2.0, device=dev), torch.full((H * d, ), 0.5, device=dev)
        sS = torch.zeros(n_seq, H, K.scan_state_floats(d, d), device=dev)
        qn, kn, vv = torch.randn(Tn, H * d, device=dev) * 0.1, torch.randn(Tn, H * d, device=dev) * 0.1, torch.randn(Tn, H * d, device=dev)
        bp, ap = torch.sigmoid(torch.randn(Tn, H, device=dev)), torch.exp(-0.08 * torch.nn.functional.softplus(torch.randn(Tn, H * d, device=dev) - 2.0))
        dS = torch.zeros(n_seq, H, K.scan_state_floats(d, d), device=dev)
        state_b = n_seq * H * d * d * 8
        add(f"tied_gate_scan ({H} x {d} x {d}), {label}", _event_ms(torch, lambda: K.tied_gate_scan(proj, 0, H * d, 2 * H * d, fb, lo, desc, n_seq, sS, H, d, d), 5, flush),
            f"delta_rule_scan ({H} x {d} x {d}; Kulanex), {label}", _event_ms(torch, lambda: K.delta_rule_scan(qn, kn, vv, bp, ap, desc, n_seq, dS, H, H, d, d), 5, flush),
            nbytes=Tn * H * d * (3 * 2 + 4) + state_b, like_bytes=Tn * H * (4 * d * 4 + 4) + Tn * H * d * 4 + state_b)
        o32, gt, og = torch.randn(Tn, H * d, device=dev), torch.randn(Tn, H * d, device=dev).to(bf), torch.empty(Tn, H * d, device=dev, dtype=bf)
        add(f"head_norm_gate without a gate, {label}", _event_ms(torch, lambda: K.head_norm_gate(o32, nw, None, og, H, d, 1e-6, shared_weight=True), 10, flush),
            f"head_norm_gate (Kulanex), {label}", _event_ms(torch, lambda: K.head_norm_gate(o32, nw, gt, og, H, d, 1e-6, shared_weight=True), 10, flush),
            nbytes=Tn * H * d * 6, like_bytes=Tn * H * d * 8)
    return rows


def run_pudinex(args):
    """Prefill and decode throughput of Pudinex through the FastGen engine at a few layer sizes, beside a Kulanex (the closest family: state
    slots beside the paged cache) and a Mixtral of equal size (same width, layers, heads, experts, ff, top-k, vocabulary), plus the isolated
    kernels of the design beside their likes."""
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.inference.v2 import RaggedInferenceEngineConfig, build_engine_from_state_dict
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    assert dist.get_world_size() == 1, "--workload pudinex is a one-GPU comparison"
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        peaks = dict(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), source="measured")
    n_seqs, prompt, budget = min(args.sequences, 64), 1024, 4096
    results, clocks, l0 = {}, None, native.launch_count
    g = torch.Generator().manual_seed(11)
    for name in (args.model.split(",") if args.model != "7b" else ["s", "m"]):
        W, L, H, d, hkv, E, top, ff, V = PUDINEX_SIZES[name]
        max_ctx = -(-(prompt + 4 * (args.steps + args.warmup) * 4 + 64) // 128) * 128
        ecfg = RaggedInferenceEngineConfig(state_manager={"max_ragged_batch_size": budget, "max_ragged_sequence_count": n_seqs, "max_tracked_sequences": n_seqs,
                                                          "max_context": max_ctx, "memory_config": {"mode": "allocate", "size": n_seqs * (max_ctx // 128) + 4}})
        res = {}
        for fam in ("pudinex", "kulanex", "mixtral"):
            if fam == "pudinex":
                cfg, sd = _pudinex_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            elif fam == "kulanex":
                cfg, sd = _kulanex_state(torch, dev, W, L, H, d, hkv, 1024, E, top, ff, V)
            else:
                cfg, sd = _mixtral_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            eng = build_engine_from_state_dict(fam, cfg, sd, ecfg, dtype=torch.bfloat16)
            n_params = sum(v.numel() for v in sd.values())
            del sd
            prompts = [torch.randint(0, V, (prompt, ), generator=g).pin_memory() for _ in range(n_seqs)]
            uids = list(range(n_seqs))
            state = {"live": False, "next": None}

            def prefill():
                if state["live"]:
                    for u in uids:
                        eng.flush(u)
                per = budget // prompt
                nxt = torch.zeros(n_seqs, dtype=torch.long)
                for i in range(0, n_seqs, per):
                    us = uids[i:i + per]
                    nxt[i:i + len(us)] = eng.put(us, [prompts[u] for u in us]).argmax(-1).cpu()
                state["live"], state["next"] = True, nxt

            def decode():
                nxt = state["next"]
                for _ in range(4):
                    nxt = eng.put(uids, [nxt[u:u + 1] for u in uids]).argmax(-1).cpu()
                state["next"] = nxt

            ms_p, _ = _timed(torch, dist, prefill, args.steps, 3)
            ms_d, clk = _timed(torch, dist, decode, args.steps, args.warmup)
            if fam == "pudinex":
                clocks = clk
            res[fam] = {"params_b": round(n_params / 1e9, 3), "prefill_tokens_per_s": round(n_seqs * prompt / ms_p * 1e3, 1), "prefill_ms": round(ms_p, 2),
                        "decode_tokens_per_s": round(n_seqs * 4 / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d / 4, 3)}
            del eng
            torch.cuda.empty_cache()
        for other in ("kulanex", "mixtral"):
            res["pudinex_over_" + other] = {"prefill": round(res["pudinex"]["prefill_tokens_per_s"] / res[other]["prefill_tokens_per_s"], 3),
                                            "decode": round(res["pudinex"]["decode_tokens_per_s"] / res[other]["decode_tokens_per_s"], 3)}
        res["shape"] = {"width": W, "layers": L, "heads": H, "head_dim": d, "kv_heads": hkv, "experts": E, "identity": PUDINEX_IDENTITY, "top": top, "ff": ff}
        res["kernels"] = _pudinex_kernel_table(torch, peaks, W, H, d, hkv, E, top, ff, 4096, 2048, n_seqs)
        results[name] = res
    launches = native.launch_count - l0
    last = results[list(results)[-1]]
    extra = {"results": results, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
             "e2e": {"value": last["pudinex"]["decode_tokens_per_s"], "unit": "generated tokens/s", "h2d_bytes_per_step": n_seqs * 8, "d2h_bytes_per_step": n_seqs * 8},
             "reference_arm": "none: the reference has no model of this design"}
    config = {"model": "pudinex (random weights) beside kulanex and mixtral of equal size", "sizes": list(results), "sequences": n_seqs, "prompt_len": prompt,
              "token_budget_per_forward": budget, "decode_steps_per_timed_step": 4, "kv_block": 128,
              "l2_policy": "engine steps: weights exceed the 126 MB L2, no flush; isolated kernels: 256 MB write before every timed run"}
    print(json.dumps(_line("generated tokens/sec Pudinex FastGen ragged decode, 1 GPU (prefill, a Kulanex and a Mixtral of equal size alongside)",
                           last["pudinex"]["decode_tokens_per_s"], "tokens/s", 1, args, last["pudinex"]["decode_ms_per_step"], config, clocks, launches, extra)),
          flush=True)


MIDULORN_SIZES = PUDINEX_SIZES  # the same widths, heads, experts and vocabularies: the twins are built from one tuple
MIDULORN_ROT = 32  # rotated entries per query head of the latent-attention layers (their latent has head_dim - 32 values: a cached row of head_dim)
MIDULORN_TAPS, MIDULORN_PART = 4, 1024


def _midulorn_state(torch, dev, W, L, H, d, hkv, E, top, ff, V):
    """Layers cycle 'latent_attention' (H heads of d - 32 plain + 32 rotated entries, values of d, latent of d - 32 beside a rotated key part of
    32: a cached row of d), 'mingru' (width H d), 'attention' (H:hkv heads of d behind 4 taps, parts of 1024, values mixed with the first such
    layer's), 'mingru'; every layer with the MoE feed-forward (E experts, top) but the last, whose feed-forward is dense (xIELU, hidden E ff / 2)."""
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    dense = {"kind": "dense", "ff": E * ff // 2}
    rot, n = MIDULORN_ROT, H * d
    lat = {"type": "latent_attention", "mixer": {"heads": H, "dim": d - rot, "rot_dim": rot, "vdim": d, "kv_rank": d - rot, "scale": d ** -0.5,
                                                 "rot": {"base": 1e6, "dims": rot}}}
    rec = {"type": "mingru", "mixer": {"width": n}}
    att = {"type": "attention", "mixer": {"heads": H, "kv_heads": hkv, "dim": d, "vdim": d, "conv": MIDULORN_TAPS, "mask": {"size": MIDULORN_PART},
                                          "scale": d ** -0.5, "v_mix": True}}
    kinds = [lat, rec, att, rec]
    layers = [dict(kinds[i % 4], mlp=dense if i == L - 1 else moe) for i in range(L)]
    cfg = {"architecture": "Midulorn", "vocab": V, "width": W, "norm": {"eps": 1e-6}, "embedding": {"scale": W ** 0.5}, "postln_alpha": 2.0,
           "logit_scale": 0.25, "layers": layers}

    def r(*shape, std=0.02, mean=0.0):
        return torch.empty(*shape, device=dev, dtype=torch.bfloat16).normal_(mean, std)

    sd = {"embed": r(V, W, std=0.05), "final.norm": r(W, mean=1.0)}
    for i, Lc in enumerate(layers):
        p, a = f"l{i}.", f"l{i}.mix."
        sd.update({p + "norm1": r(W, mean=1.0), p + "norm2": r(W, mean=1.0)})
        if Lc["mlp"]["kind"] == "moe":
            sd[p + "mlp.router"] = r(E, W, std=0.5)
            for e in range(E):
                sd.update({p + f"mlp.e{e}.gate": r(ff, W), p + f"mlp.e{e}.up": r(ff, W), p + f"mlp.e{e}.down": r(W, ff)})
        else:
            sd.update({p + "mlp.up": r(dense["ff"], W), p + "mlp.down": r(W, dense["ff"]), p + "mlp.act": r(2, std=0.5)})
        if Lc["type"] == "latent_attention":
            sd.update({a + "q": r(H * d, W), a + "dkv": r(d, W), a + "dkv.norm": r(d - rot, mean=1.0), a + "uk": r(H * (d - rot), d - rot, std=0.1),
                       a + "uv": r(H * d, d - rot, std=0.1), a + "sink": r(H, std=1.0), a + "g": r(H, W), a + "o": r(W, H * d)})
        elif Lc["type"] == "mingru":
            sd.update({a + "z": r(n, W), a + "z.b": r(n, mean=-1.0, std=1.0), a + "x": r(n, W), a + "x.b": r(n), a + "g": r(n, W), a + "o": r(W, n)})
        else:
            for nm, c in (("q", H * d), ("k", hkv * d), ("v", hkv * d)):
                sd.update({a + nm: r(c, W), a + nm + ".b": r(c), a + nm + ".conv": r(c, MIDULORN_TAPS, std=0.5)})
            sd.update({a + "q.norm": r(d, mean=1.0), a + "k.norm": r(d, mean=1.0), a + "vmix": r(1, mean=0.3, std=0.0).reshape(()), a + "r1": r(H, mean=1.0, std=0.1),
                       a + "r2": r(H, mean=0.5, std=0.05), a + "sink": r(H, std=1.0), a + "o": r(W, H * d), a + "o.b": r(W)})
    return cfg, sd


def _midulorn_kernel_table(torch, peaks, W, H, d, hkv, E, top, ff, T, ctx, n_dec):
    """Every kernel of the design beside the like kernel of the closest family (Pudinex; Linasun for the latent rows, Kulanex for the convolving
    prepare), isolated, with the fraction of the measured roofline (HBM copy bandwidth for the streaming kernels, cuBLAS bf16 rate for attention
    prefill)."""
    from deepspeedsyclsupport_b200.inference.v2 import kernels as K
    from deepspeedsyclsupport_b200.ops import fused_ops as FO
    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = []

    def add(name, ms, like, like_ms, nbytes=None, like_bytes=None, flops=None, like_flops=None):
        def frac(ms_, b, f):
            return round(max((b or 0) / hbm, (f or 0) / tf) / (ms_ * 1e-3), 3)
        rows.append({"kernel": name, "ms": round(ms, 4), "roofline_frac": frac(ms, nbytes, flops), "like": like, "like_ms": round(like_ms, 4),
                     "like_roofline_frac": frac(like_ms, like_bytes if like_bytes is not None else nbytes, like_flops if like_flops is not None else flops)})

    rot, n = MIDULORN_ROT, H * d
    x32, y, y32, g32 = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev), torch.randn(W, device=dev)
    add("post_sum_norm (bf16 branch + bias in; fp32 stream and bf16 copy out)", _event_ms(torch, lambda: K.post_sum_norm(x32, y, g32, 2.0, 1e-6, bias=g32), 20, flush),
        "stream_group_norm (2 parts; bf16 branch in, bf16 out; Pudinex)", _event_ms(torch, lambda: K.stream_group_norm(x32, (y, ), None, g32, 2, 1e-6), 20, flush),
        nbytes=T * W * (4 + 2 + 4 + 2))
    add("post_sum_norm (fp32 branch of the experts in)", _event_ms(torch, lambda: K.post_sum_norm(x32, None, g32, 2.0, 1e-6, y32=y32), 20, flush),
        "stream_group_norm (fp32 branch in; Pudinex)", _event_ms(torch, lambda: K.stream_group_norm(x32, (), y32, g32, 2, 1e-6), 20, flush),
        nbytes=T * W * (4 + 4 + 4 + 2))
    F = E * ff // 2
    up, gpair, coef = torch.randn(T, F, device=dev).to(bf), torch.randn(T, 2 * F, device=dev).to(bf), K.xielu_coefficients(0.3, -0.2).to(dev)
    add("xielu", _event_ms(torch, lambda: K.xielu(up, coef), 20, flush), "gated_act (silu; Mixtral)", _event_ms(torch, lambda: FO.gated_act(gpair, "silu"), 20, flush),
        nbytes=T * F * 4, like_bytes=T * F * 6)
    lg = torch.randn(T, E, device=dev)
    add("grouped_topk_gating (softmax, not renormalised)", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top), 20, flush),
        "grouped_topk_gating (softmax, renormalised; Pudinex)", _event_ms(torch, lambda: K.grouped_topk_gating(lg, top, normalize=True), 20, flush),
        nbytes=T * (E * 4 + top * 12))
    a3, gh, gfull = torch.randn(H, T, d, device=dev).to(bf), torch.randn(T, H, device=dev).to(bf), torch.randn(T, H * d, device=dev).to(bf)
    add("gate_heads_scalar (one gate per token and head)", _event_ms(torch, lambda: K.gate_heads_scalar(a3, gh), 20, flush),
        "gate_heads (one gate per value; Linasun)", _event_ms(torch, lambda: K.gate_heads(a3, gfull), 20, flush), nbytes=T * n * 4, like_bytes=T * n * 6)
    bs = 128
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import RampRotaryScalingConfig
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.sink_blocked_attention import ramp_scaled_frequencies
    pfreq, pmag = ramp_scaled_frequencies(d // 2, 1e6, RampRotaryScalingConfig(factor=8.0, original=8192, fast=32.0, slow=1.0))
    pfreq = pfreq.to(dev)
    lfreq = torch.tensor([1e6 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64, device=dev)
    Hp = 1 << (H - 1).bit_length()
    for label, n_seq, new, seen in (("prefill", max(1, T // 2048), min(T, 2048), ctx), ("decode", n_dec, 1, ctx)):
        per = -(-(seen + new) // bs)
        nb = n_seq * per
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(n_seq, per)
        tok_seq = torch.arange(n_seq, dtype=torch.int32, device=dev).repeat_interleave(new)
        tok_pos = (seen + torch.arange(new, dtype=torch.int32, device=dev)).repeat(n_seq)
        desc = torch.tensor([[i * new, new, seen, i] for i in range(n_seq)], dtype=torch.int32, device=dev)
        Tn = n_seq * new
        dec = label == "decode"
        kv = torch.randn(nb, 2, bs, hkv, d, device=dev).to(bf)
        qkv = torch.randn(Tn, (H + 2 * hkv) * d, device=dev).to(bf)
        nw = torch.randn(d, device=dev)
        qo = torch.empty(Tn, H * d, device=dev, dtype=bf)
        planes = K.cache_planes(kv)
        C = (H + 2 * hkv) * d
        cw, cb, mix = torch.randn(MIDULORN_TAPS, C, device=dev), torch.randn(C, device=dev), torch.full((1, ), 0.3, device=dev)
        cstate = torch.zeros(n_seq, MIDULORN_TAPS - 1, C, device=dev, dtype=bf)
        vsrc = torch.randn(Tn, hkv * d, device=dev).to(bf)

        def cprep():
            K.conv_head_norm_append(qkv, 0, cb, cw, nw, nw, cstate, desc, tok_seq, tok_pos, bt, bs, planes[0], planes[1], qo, H, hkv, d, d, MIDULORN_TAPS, 1e-6,
                                    v_other=vsrc, mix=mix)
            K.conv_state_update(qkv, 0, C, cstate, 0, desc, n_seq, MIDULORN_TAPS)
        add(f"conv_head_norm_append + conv_state_update, {label}", _event_ms(torch, cprep, 10, flush), f"head_norm_rotary_append (Pudinex), {label}",
            _event_ms(torch, lambda: K.head_norm_rotary_append(qkv, 0, H * d, (H + hkv) * d, nw, nw, pfreq, pmag, tok_seq, tok_pos, bt, bs, planes[0], planes[1], qo,
                                                               H, hkv, d, d, d // 2, 1e-6), 10, flush),
            nbytes=Tn * (C * 4 + hkv * d * 2), like_bytes=Tn * C * 4)
        keys = n_seq * new * (seen + (new + 1) / 2)
        out = torch.empty(Tn, H * d, device=dev, dtype=bf)
        abytes = n_seq * (seen + new) * hkv * d * 4 + Tn * H * d * 4
        r1, r2, sk = torch.full((H, ), 1.0, device=dev), torch.full((H, ), 0.5, device=dev), torch.randn(H, device=dev)
        ms_like = _event_ms(torch, lambda: K.paged_flash_sink(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, d ** -0.5, 50.0, 1.0, decode=dec), 10, flush)
        add(f"attention, distance term + learned sinks, one part, tcgen05, {label} (GQA {H}:{hkv})",
            _event_ms(torch, lambda: K.paged_flash_sink(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, d ** -0.5, 0.0, 0.0, decode=dec, sink_logit=sk, r1=r1, r2=r2,
                                                        part=1 << 20), 10, flush),
            f"attention, soft cap 50 + sink, tcgen05, {label} (Pudinex)", ms_like, nbytes=abytes, flops=4.0 * keys * H * d)
        # parts of 1024: a query sees at most its own part, so the kernel visits a fraction of the pages (the work shrinks with it)
        pk = n_seq * sum(min(p % MIDULORN_PART + 1, p + 1) for p in range(seen, seen + new))
        pbytes = n_seq * min(seen + new, MIDULORN_PART + new) * hkv * d * 4 + Tn * H * d * 4
        add(f"attention, distance term + learned sinks, parts of {MIDULORN_PART}, tcgen05, {label}",
            _event_ms(torch, lambda: K.paged_flash_sink(qo, kv, tok_seq, tok_pos, bt, out, H, hkv, d, d ** -0.5, 0.0, 0.0, decode=dec, sink_logit=sk, r1=r1, r2=r2,
                                                        part=MIDULORN_PART), 10, flush),
            f"attention, soft cap 50 + sink, tcgen05, {label} (Pudinex; whole context)", ms_like, nbytes=pbytes, like_bytes=abytes, flops=4.0 * pk * H * d,
            like_flops=4.0 * keys * H * d)
        # low-rank rows: rotation + norm + append, then one-plane attention with sinks, beside the same without rotation / sinks
        lat = torch.randn(Tn, H * d + d + H, device=dev).to(bf)
        lcache = torch.randn(nb, bs, d, device=dev).to(bf)
        wkv = torch.randn(d - rot, device=dev)
        lat2 = torch.randn(Tn, 2 * d, device=dev).to(bf)
        wq2 = torch.randn(d, device=dev)
        add(f"latent_rotary_append, {label}", _event_ms(torch, lambda: K.latent_rotary_append(lat, 0, H * d, wkv, lfreq, tok_seq, tok_pos, bt, lcache, H, d - rot, rot,
                                                                                            d - rot, rot, 1e-6), 10, flush),
            f"latent_norm_append (Linasun), {label}", _event_ms(torch, lambda: K.latent_norm_append(lat2, wq2, wq2, lcache, tok_seq, tok_pos, bt, d, d, 1e-6), 10, flush),
            nbytes=Tn * (H * rot * 4 + d * 4), like_bytes=Tn * d * 8)
        qa = torch.randn(Hp, Tn, d, device=dev).to(bf)
        skp = torch.randn(Hp, device=dev)
        lbytes = n_seq * (seen + new) * d * 2 + Tn * Hp * d * 4
        add(f"latent attention with learned sinks, tcgen05 one-plane, {label} ({Hp} heads)",
            _event_ms(torch, lambda: K.paged_latent_flash(qa.transpose(0, 1), lcache, tok_seq, tok_pos, bt, d ** -0.5, decode=dec, heads=Hp, sink_logit=skp), 10, flush),
            f"latent attention, tcgen05 one-plane, {label} (Linasun)",
            _event_ms(torch, lambda: K.paged_latent_flash(qa.transpose(0, 1), lcache, tok_seq, tok_pos, bt, d ** -0.5, decode=dec, heads=Hp), 10, flush),
            nbytes=lbytes, flops=4.0 * keys * Hp * d)
        # the recurrence beside Pudinex's scan: one number of state per channel against a d x d matrix per head
        proj = torch.randn(Tn, 3 * n, device=dev).to(bf)
        zb = torch.zeros(n, device=dev)
        sS = torch.zeros(n_seq, n, device=dev)
        og = torch.empty(Tn, n, device=dev, dtype=bf)
        fb, lo = torch.full((n, ), 2.0, device=dev), torch.full((n, ), 0.5, device=dev)
        tS = torch.zeros(n_seq, H, K.scan_state_floats(d, d), device=dev)
        ms_like = _event_ms(torch, lambda: K.tied_gate_scan(proj, 0, n, 2 * n, fb, lo, desc, n_seq, tS, H, d, d), 5, flush)
        add(f"mingru_scan (width {n}), {label}", _event_ms(torch, lambda: K.mingru_scan(proj, 0, n, 2 * n, zb, zb, tok_seq, desc, n_seq, sS, og, n), 10, flush),
            f"tied_gate_scan ({H} x {d} x {d}; Pudinex), {label}", ms_like, nbytes=Tn * n * (3 * 2 + 2) + n_seq * n * 8,
            like_bytes=Tn * n * (3 * 2 + 4) + n_seq * H * d * d * 8)
        if not dec:
            add(f"mingru_scan as one walk per sequence (width {n}), {label}",
                _event_ms(torch, lambda: K.mingru_scan(proj, 0, n, 2 * n, zb, zb, tok_seq, desc, n_seq, sS, og, n, pieces=False), 5, flush),
                f"tied_gate_scan ({H} x {d} x {d}; Pudinex), {label}", ms_like, nbytes=Tn * n * (3 * 2 + 2) + n_seq * n * 8,
                like_bytes=Tn * n * (3 * 2 + 4) + n_seq * H * d * d * 8)
    return rows


def run_midulorn(args):
    """Prefill and decode throughput of Midulorn through the FastGen engine at a few layer sizes, beside a Pudinex (the closest family: attention
    with sinks on per-head normed queries and keys, recurrent layers in the state slots, softmax router) and a Mixtral of equal size (same width,
    layers, heads, experts, ff, top-k, vocabulary), plus the isolated kernels of the design beside their likes."""
    sys.path.insert(0, ROOT)
    import torch
    import deepspeedsyclsupport_b200 as deepspeed
    from deepspeedsyclsupport_b200 import comm as dist
    from deepspeedsyclsupport_b200.inference.v2 import RaggedInferenceEngineConfig, build_engine_from_state_dict
    from deepspeedsyclsupport_b200.ops import native
    deepspeed.init_distributed()
    assert dist.get_world_size() == 1, "--workload midulorn is a one-GPU comparison"
    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        peaks = dict(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), source="measured")
    n_seqs, prompt, budget = min(args.sequences, 64), 1024, 4096
    results, clocks, l0 = {}, None, native.launch_count
    g = torch.Generator().manual_seed(11)
    for name in (args.model.split(",") if args.model != "7b" else ["s", "m"]):
        W, L, H, d, hkv, E, top, ff, V = MIDULORN_SIZES[name]
        max_ctx = -(-(prompt + 4 * (args.steps + args.warmup) * 4 + 64) // 128) * 128
        ecfg = RaggedInferenceEngineConfig(state_manager={"max_ragged_batch_size": budget, "max_ragged_sequence_count": n_seqs, "max_tracked_sequences": n_seqs,
                                                          "max_context": max_ctx, "memory_config": {"mode": "allocate", "size": n_seqs * (max_ctx // 128) + 4}})
        res = {}
        for fam in ("midulorn", "pudinex", "mixtral"):
            if fam == "midulorn":
                cfg, sd = _midulorn_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            elif fam == "pudinex":
                cfg, sd = _pudinex_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            else:
                cfg, sd = _mixtral_state(torch, dev, W, L, H, d, hkv, E, top, ff, V)
            eng = build_engine_from_state_dict(fam, cfg, sd, ecfg, dtype=torch.bfloat16)
            n_params = sum(v.numel() for v in sd.values())
            del sd
            prompts = [torch.randint(0, V, (prompt, ), generator=g).pin_memory() for _ in range(n_seqs)]
            uids = list(range(n_seqs))
            state = {"live": False, "next": None}

            def prefill():
                if state["live"]:
                    for u in uids:
                        eng.flush(u)
                per = budget // prompt
                nxt = torch.zeros(n_seqs, dtype=torch.long)
                for i in range(0, n_seqs, per):
                    us = uids[i:i + per]
                    nxt[i:i + len(us)] = eng.put(us, [prompts[u] for u in us]).argmax(-1).cpu()
                state["live"], state["next"] = True, nxt

            def decode():
                nxt = state["next"]
                for _ in range(4):
                    nxt = eng.put(uids, [nxt[u:u + 1] for u in uids]).argmax(-1).cpu()
                state["next"] = nxt

            ms_p, _ = _timed(torch, dist, prefill, args.steps, 3)
            ms_d, clk = _timed(torch, dist, decode, args.steps, args.warmup)
            if fam == "midulorn":
                clocks = clk
            res[fam] = {"params_b": round(n_params / 1e9, 3), "prefill_tokens_per_s": round(n_seqs * prompt / ms_p * 1e3, 1), "prefill_ms": round(ms_p, 2),
                        "decode_tokens_per_s": round(n_seqs * 4 / ms_d * 1e3, 1), "decode_ms_per_step": round(ms_d / 4, 3)}
            del eng
            torch.cuda.empty_cache()
        for other in ("pudinex", "mixtral"):
            res["midulorn_over_" + other] = {"prefill": round(res["midulorn"]["prefill_tokens_per_s"] / res[other]["prefill_tokens_per_s"], 3),
                                             "decode": round(res["midulorn"]["decode_tokens_per_s"] / res[other]["decode_tokens_per_s"], 3)}
        res["shape"] = {"width": W, "layers": L, "heads": H, "head_dim": d, "kv_heads": hkv, "experts": E, "top": top, "ff": ff, "rotated": MIDULORN_ROT,
                        "taps": MIDULORN_TAPS, "part": MIDULORN_PART}
        res["kernels"] = _midulorn_kernel_table(torch, peaks, W, H, d, hkv, E, top, ff, 4096, 2048, n_seqs)
        results[name] = res
    launches = native.launch_count - l0
    last = results[list(results)[-1]]
    extra = {"results": results, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
             "e2e": {"value": last["midulorn"]["decode_tokens_per_s"], "unit": "generated tokens/s", "h2d_bytes_per_step": n_seqs * 8, "d2h_bytes_per_step": n_seqs * 8},
             "reference_arm": "none: the reference has no model of this design"}
    config = {"model": "midulorn (random weights) beside pudinex and mixtral of equal size", "sizes": list(results), "sequences": n_seqs, "prompt_len": prompt,
              "token_budget_per_forward": budget, "decode_steps_per_timed_step": 4, "kv_block": 128,
              "l2_policy": "engine steps: weights exceed the 126 MB L2, no flush; isolated kernels: 256 MB write before every timed run"}
    print(json.dumps(_line("generated tokens/sec Midulorn FastGen ragged decode, 1 GPU (prefill, a Pudinex and a Mixtral of equal size alongside)",
                           last["midulorn"]["decode_tokens_per_s"], "tokens/s", 1, args, last["midulorn"]["decode_ms_per_step"], config, clocks, launches, extra)),
          flush=True)


WORKLOADS = {"fastgen70b": run_fastgen70b, "mixtral": run_mixtral, "ulysses13b": run_ulysses13b, "linasun": run_linasun, "kulanex": run_kulanex, "pudinex": run_pudinex, "midulorn": run_midulorn}
