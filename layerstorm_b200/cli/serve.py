"""``python -m layerstorm_b200.cli.serve`` - boot an engine and serve the OpenAI-compatible API.

Boot order: parse flags -> load / autoconfigure the config -> tokenizer -> engine (one process per
GPU; rank 0 owns the HTTP server, the other ranks follow its step commands) -> orchestrator thread ->
uvicorn.  ``--test-engine`` swaps the GPU engine for the deterministic null engine, so the whole
serving stack can be exercised on a machine without a GPU.
Flag surface follows the reference CLI (python/cli/serve.py:110-217).
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import threading
from typing import Any, Optional

from ..config import ConfigError, apply_env, fill_model_from_checkpoint, load_config, model_config_from, parse_pin
from ..models.config import PRESETS as MODEL_PRESETS, ModelConfig, get_preset

log = logging.getLogger("layerstorm_b200.serve")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="layerstorm_b200.cli.serve", description="OpenAI-compatible server for MLA-family MoE models on B200")
    src = p.add_argument_group("configuration source")
    src.add_argument("--config", help="engine configuration JSON")
    src.add_argument("--autoconfig", action="store_true", help="derive the configuration from the model and this machine")
    src.add_argument("--model", help="checkpoint path (HF safetensors directory or .gguf file) or a built-in shape preset: " + ", ".join(MODEL_PRESETS))
    src.add_argument("--accuracy", choices=["compact", "standard", "high", "superior"], default=None, help="autoconfig: floor of the attention-backend ladder")
    src.add_argument("--prefer", choices=["speed", "balanced", "capacity"], default=None, help="autoconfig: sort key over feasible configurations")
    src.add_argument("--pin", action="append", default=[], metavar="PATH=VALUE|FILE.json", help="autoconfig: hard constraint (repeatable)")
    src.add_argument("--autoconfig-redetect", action="store_true", help="ignore a stored autoconfig result and probe the machine again")
    src.add_argument("--vram-expert-ratio", type=float, default=None, help="autoconfig lever: fraction of owned experts resident in HBM")
    src.add_argument("--total-active-context-tokens", type=int, default=None, help="autoconfig lever: concurrency x sequence length")
    srv = p.add_argument_group("serving")
    srv.add_argument("--host", default=None)
    srv.add_argument("--port", type=int, default=None)
    srv.add_argument("--model-name", default=None, help="id reported by /v1/models")
    srv.add_argument("--tokenizer-path", default=None)
    srv.add_argument("--tokenizer-mode", default=None, choices=["auto", "hf", "byte"])
    srv.add_argument("--max-concurrent", type=int, default=None)
    srv.add_argument("--max-queued-requests", type=int, default=None)
    srv.add_argument("--sse-heartbeat-seconds", type=float, default=None)
    srv.add_argument("--max-sequence-length", type=int, default=None)
    srv.add_argument("--tool-call-parser", default=None)
    srv.add_argument("--enable-auto-tool-choice", action="store_true", default=None)
    srv.add_argument("--reasoning-parser", default=None)
    srv.add_argument("--reasoning-config", default=None, help="JSON string or file with the reasoning parser's settings")
    eng = p.add_argument_group("engine")
    eng.add_argument("--speculation-depth", type=int, default=None, help="draft tokens per speculative round (0 = off)")
    eng.add_argument("--cycle-budget-us", type=int, default=None, help="orchestrator idle poll period")
    eng.add_argument("--random-weights", action="store_true", help="random-init weights of the configured shape (benchmarks, smoke tests)")
    eng.add_argument("--kv-format", default=None, choices=["fp8", "bf16", "tq4"])
    eng.add_argument("--log-level", default="info", choices=["debug", "info", "warning", "error"])
    eng.add_argument("--test-engine", action="store_true", help="serve from the null engine (no GPU, deterministic tokens)")
    eng.add_argument("--dry-run", action="store_true", help="resolve and print the configuration, then exit")
    return p


_FLAG_TO_PATH = {
    "host": "serving.host", "port": "serving.port", "model_name": "serving.model_name", "tokenizer_path": "serving.tokenizer_path",
    "tokenizer_mode": "serving.tokenizer_mode", "max_concurrent": "serving.max_concurrent_requests",
    "max_queued_requests": "serving.max_queued_requests", "sse_heartbeat_seconds": "serving.sse_heartbeat_seconds",
    "max_sequence_length": "serving.max_sequence_length", "tool_call_parser": "serving.tool_call_parser",
    "enable_auto_tool_choice": "serving.enable_auto_tool_choice", "reasoning_parser": "serving.reasoning_parser",
    "reasoning_config": "serving.reasoning_config",
}


def overrides_from_args(args: argparse.Namespace) -> dict[str, Any]:
    out = {}
    for flag, path in _FLAG_TO_PATH.items():
        v = getattr(args, flag, None)
        if v is not None:
            out[path] = v
    if args.speculation_depth is not None:
        out["speculation.enabled"] = args.speculation_depth > 0
        out["speculation.mtp.max_depth"] = max(1, args.speculation_depth)
    return out


def collect_pins(items: list[str]) -> dict[str, Any]:
    pins: dict[str, Any] = {}
    for it in items:
        if it.endswith(".json") and os.path.exists(it):
            pins.update(json.load(open(it)))
        else:
            k, v = parse_pin(it)
            pins[k] = v
    return pins


def resolve_model(args: argparse.Namespace, cfg: Optional[dict]) -> tuple[Optional[ModelConfig], Optional[str]]:
    """(shape, checkpoint path).  ``--model`` wins over ``model.weights_path``."""
    src = args.model or (cfg or {}).get("model", {}).get("weights_path") or None
    if src and src.lower() in MODEL_PRESETS:
        return get_preset(src), None
    if src and os.path.exists(src):
        from ..models.config import from_hf_config
        d = src if os.path.isdir(src) else os.path.dirname(src)
        cj = os.path.join(d, "config.json")
        if os.path.exists(cj):
            return from_hf_config(cj), src
        if src.endswith(".gguf") or os.path.isdir(src):
            from ..autoconfig.modelprobe import probe
            try:
                return probe(src).shape, src                     # GGUF metadata carries the shape
            except ValueError:
                pass
        return None, src
    if src:
        raise ConfigError([f"--model: '{src}' is neither a path nor one of the built-in shapes {sorted(MODEL_PRESETS)}"])
    return None, None


def resolve_config(args: argparse.Namespace) -> tuple[dict, ModelConfig, Optional[str], Optional[str]]:
    """Returns (config, model shape, checkpoint path or None, autoconfig explanation or None)."""
    over = overrides_from_args(args)
    base = json.load(open(args.config)) if args.config else None
    shape, ckpt = resolve_model(args, base)
    explain = None
    if args.autoconfig or (base or {}).get("autoconfig", {}).get("enabled"):
        from ..autoconfig import Levers, detect, explain_text, solve, synthetic, write_result
        if shape is None:
            raise ConfigError(["--autoconfig needs --model (a checkpoint with config.json or a built-in shape)"])
        ac = (base or {}).get("autoconfig", {})
        stored = ac.get("output_path") or ""
        hw = detect((base or {}).get("hardware", {}).get("nvme_paths"))
        if not hw.gpus and args.test_engine:
            hw = synthetic(1)
        if stored and os.path.exists(stored) and not args.autoconfig_redetect:
            prev = json.load(open(stored))
            if prev.get("autoconfig", {}).get("fingerprint") == hw.fingerprint():
                log.info("reusing the stored autoconfig result %s", stored)
                cfg = load_config(prev, over)
                return apply_env(cfg), model_config_from(cfg), ckpt, "stored result reused"
        lv = Levers(vram_expert_ratio=args.vram_expert_ratio if args.vram_expert_ratio is not None else ac.get("vram_expert_ratio"),
                    total_active_context_tokens=args.total_active_context_tokens or ac.get("total_active_context_tokens"),
                    prefer=args.prefer or ac.get("prefer", "balanced"), accuracy=args.accuracy or ac.get("accuracy", "standard"))
        pins = collect_pins(args.pin)
        for k in ("serving.max_concurrent_requests", "serving.max_sequence_length"):
            if k in over:
                pins.setdefault(k, over[k])
        res = solve(shape, hw, lv, pins, base)
        explain = explain_text(res)
        if stored:
            write_result(res, stored)
        cfg = load_config(res.config, over)
    else:
        cfg = load_config(base, over)
        if ckpt:
            cfg["model"]["weights_path"] = ckpt
            cfg["model"]["weights_format"] = "gguf" if ckpt.endswith(".gguf") else "safetensors"
        cfg = fill_model_from_checkpoint(cfg)
        if shape is None:
            shape = model_config_from(cfg)
    return apply_env(cfg), shape, ckpt, explain


def build_engine(cfg: dict, shape: ModelConfig, ckpt: Optional[str], args: argparse.Namespace):
    sv = cfg["serving"]
    page = cfg["memory"]["kv_cache"]["page_size_tokens"]
    if args.test_engine:
        from ..runtime.null_engine import NullEngine
        return NullEngine(vocab=max(512, min(shape.vocab, 65536)), max_seqs=sv["max_concurrent_requests"] + 4,
                          max_ctx=sv["max_sequence_length"], page=page)
    import torch
    from ..models.device_model import DeviceModel
    from ..runtime.engine import Engine
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is visible; use --test-engine to serve from the null engine")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        # one process per GPU (torchrun): tensor / expert parallel model shards, in-kernel NVLink collectives
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    kv_fmt = args.kv_format or {"fp8_e4m3": "fp8", "bf16": "bf16", "fp16": "bf16", "turboquant4": "tq4"}.get(cfg["quantization"]["kv_cache"], "fp8")
    want_mtp = bool(cfg["speculation"]["enabled"]) and cfg["speculation"]["method"] == "mtp"      # load the MTP block only when it drafts
    # a derived configuration that keeps only part of every GPU's experts in HBM (autoconfig.vram_expert_ratio < 1): the rest lives in
    # pinned host memory and streams into the slots; the model is loaded layer by layer so that it never has to fit in HBM as a whole
    streamer = None
    ratio = float((cfg.get("autoconfig") or {}).get("vram_expert_ratio") or 1.0)
    if ratio < 1.0 and shape.n_routed > 0:
        if world > 1:
            log.warning("expert streaming is wired for one GPU per model; autoconfig.vram_expert_ratio = %.2f ignored with %d ranks", ratio, world)
        else:
            from ..runtime.streaming import ExpertStreamer
            e_total = shape.n_routed + shape.n_shared
            slots = max(shape.top_k + shape.n_shared, min(e_total, int(ratio * e_total)))
            live = None
            if ckpt and not args.random_weights and str(ckpt).endswith(".gguf") and shape.expert_quant == "gguf":
                # a GGUF checkpoint: slot images of natively readable layers go from the file straight into the pinned store
                from ..models.checkpoint import open_checkpoint
                from ..runtime.live_gguf import LiveGgufExpertSource
                try:
                    live = LiveGgufExpertSource(open_checkpoint(ckpt, shape)[1], shape, threads=cfg["preprocessing"]["live_prepack_threads"] or 8)
                except ValueError as e:
                    log.warning("live GGUF expert source unavailable: %s", e)
            streamer = ExpertStreamer(None, slots_per_layer=slots, prefetch=True, cfg=shape, device=dev,
                                      place_freq=cfg["memory"]["arena_placement"]["freq_table"] or None, live_source=live)
            log.info("expert cache: %d of %d expert slots per MoE layer in HBM, the rest streams from pinned host memory", slots, e_total)
    hook = streamer.add_layer if streamer is not None else None
    if ckpt and not args.random_weights:
        from ..models.checkpoint import open_checkpoint
        _, w = open_checkpoint(ckpt, shape)
        model = DeviceModel.from_state_dict(shape, w, dev, kv_fmt, page, tp_rank=rank, tp_size=world, with_mtp=want_mtp, layer_hook=hook,
                                            skip_experts=streamer.covers if (streamer is not None and streamer.live_source is not None) else None)
    else:
        log.warning("serving RANDOM weights of shape %s", shape.name)
        model = DeviceModel.random_init(shape, dev, kv_fmt, page, expert_slots="auto", embed_on_host=shape.vocab * shape.hidden > (1 << 28),
                                        tp_rank=rank, tp_size=world, with_mtp=want_mtp, layer_hook=hook)
    if streamer is not None:
        streamer.attach(model)
        streamer.configure_eviction(cfg["memory"]["expert_cache"])
    max_ctx = sv["max_sequence_length"]
    if world > 1:
        from ..parallel.symm import PeerComm
        chunk_rows = max(4, cfg["orchestrator"]["prefill_chunk_tokens"], cfg["orchestrator"]["max_batch_size"])
        model.attach_comm(PeerComm(chunk_rows * shape.hidden, dev), PeerComm(2 * max(4, cfg["orchestrator"]["max_batch_size"]), dev))
        pc_on = sv["prefix_cache"]["enabled"] and sv["prefix_cache"]["max_entries"] > 0
        if cfg["hardware"].get("dcp_kv_mode") == "sharded" and cfg["hardware"].get("dcp_enabled", True) and not pc_on and not cfg["speculation"]["enabled"]:
            # context-parallel KV shards (no fork / rewind in this mode, hence only without prefix cache and speculation)
            from ..parallel.dcp import DcpAttention
            model.enable_dcp(DcpAttention(shape.n_heads, shape.kv_lora, shape.qk_rope, max_rows=chunk_rows, device=dev,
                                          chunk=int(cfg["memory"]["kv_cache"].get("dcp_chunk_size", 64))))
    pages = cfg["memory"]["kv_cache"]["max_pages_per_gpu"]
    eng = Engine(model, max_seqs=sv["max_concurrent_requests"] + 4, max_ctx=max_ctx,
                 prefill_chunk=cfg["orchestrator"]["prefill_chunk_tokens"],
                 max_batch=max(1, min(32, cfg["orchestrator"]["max_batch_size"], sv["max_concurrent_requests"])),
                 num_pages=None if pages in ("auto", None) else int(pages),
                 use_graph=cfg["compute"]["cuda_graphs"]["enabled"] and streamer is None)      # a streamed layer has a host wait: eager steps
    return eng


def prefill_slice_factor(cfg: dict) -> int:
    """Engine chunks per prefill slice of a joining request (continuous batching: the running requests wait for one slice between two
    of their decode steps).  ``orchestrator.performance_objective`` decides: the more weight on throughput, the longer the slices (fewer
    interruptions of the prefill), the more on latency, the shorter (the default 0.6 / 0.4 gives four chunks)."""
    from ..speculation.policies import PerformanceObjective
    po = PerformanceObjective.from_config(cfg)
    return max(1, min(16, int(round(10 * po.throughput_weight))))


def build_block_draft(cfg: dict, shape: ModelConfig, target, args: argparse.Namespace):
    """The DSpark block draft (``speculation/dspark.py``) when ``speculation.dspark.checkpoint_path`` is a speculators-format dspark
    checkpoint, or - without a checkpoint - when ``speculation.dspark.aux_hidden_state_layer_ids`` is set (RANDOM draft weights of a
    small geometry: plumbing and timing runs).  None when neither applies or the engine cannot report aux hidden states."""
    from ..speculation import dspark as dsp
    ds = cfg["speculation"]["dspark"]
    path = ds["checkpoint_path"]
    if path and not dsp.is_dspark_checkpoint(path):
        return None
    if not path and not ds["aux_hidden_state_layer_ids"]:
        return None
    if not hasattr(target, "enable_aux_capture") or int(os.environ.get("WORLD_SIZE", 1)) > 1:
        log.warning("the block draft needs an engine that reports aux hidden states (one GPU); serving without it")
        return None
    import torch
    if path:
        dcfg, tensors = dsp.load_dspark_checkpoint(path)
        for key, have in (("block_size", dcfg.block_size), ("markov_rank", dcfg.markov_rank), ("mask_token_id", dcfg.mask_token_id),
                          ("draft_vocab_size", dcfg.draft_vocab_size), ("aux_hidden_state_layer_ids", dcfg.aux_hidden_state_layer_ids)):
            if ds[key] and ds[key] != have:
                log.warning("speculation.dspark.%s = %s, the checkpoint says %s: the checkpoint's value is used", key, ds[key], have)
    else:
        dcfg = dsp.draft_config_for_target(shape.hidden, shape.vocab, shape.n_layers, block_size=ds["block_size"], markov_rank=min(ds["markov_rank"], 64))
        dcfg.aux_hidden_state_layer_ids = [int(l) for l in ds["aux_hidden_state_layer_ids"]]
        log.warning("speculation.dspark.checkpoint_path is empty: RANDOM block-draft weights (%d layers, aux layers %s)", dcfg.num_hidden_layers,
                    dcfg.aux_hidden_state_layer_ids)
        tensors = dsp.random_dspark_tensors(dcfg, 0)
    dev = torch.device("cuda", int(ds["draft_gpus"][0])) if ds["draft_gpus"] else target.dev
    cap = min(cfg["serving"]["max_sequence_length"], max(ds["draft_context_capacity_tokens"], 4 * dcfg.block_size))
    try:
        # on the GPU the draft's matrices are stored as speculation.dspark.draft_weights_quant and applied by the framework's own kernels
        # (LSB_DSPARK_TORCH_GEMM=1: library GEMMs over bf16 tensors instead)
        kernels = ds["draft_weights_quant"] if dev.type == "cuda" and os.environ.get("LSB_DSPARK_TORCH_GEMM", "0") != "1" else None
        bb = dsp.DsparkBackbone(dcfg, tensors, dev, torch.bfloat16, ctx_capacity=cap, rotate=ds["ctx_rotate"], kernels=kernels)
        draft = dsp.DeviceDsparkDraft(target, bb, {"speculative_tokens": ds["speculative_tokens"], "confidence_enabled": ds["confidence_enabled"] and dcfg.enable_confidence_head,
                                                  "confidence_threshold": ds["confidence_threshold"], "scheduler_mode": ds["scheduler_mode"],
                                                  "sts_temperatures": ds["sts_temperatures"]},
                                     max_contexts=int(os.environ.get("LSB_DSPARK_CONTEXTS", "4")), output_of_layer=os.environ.get("LSB_DSPARK_AUX_OUTPUT", "0") == "1")
        from ..speculation.epm_corpus import CorpusWriter, effective_dump_dir
        dump = effective_dump_dir(ds["epm_dump_dir"])
        if dump:
            # feature side of the expert-routing prediction corpus (block records + verdicts); the label side (router logits per
            # position) is recorded by the CPU reference path only
            draft.attach_corpus(CorpusWriter(dump))
            log.info("block records of the draft go to %s", dump)
        return draft
    except (NotImplementedError, ValueError) as e:
        log.warning("block draft unavailable (%s); serving without it", e)
        return None


def build_model_draft(cfg: dict, shape: ModelConfig, engine, args: argparse.Namespace):
    """(draft, depth) for the model-backed speculation methods.
    ``self_speculative``: the target drafts for itself with ``speculation.self_speculative.draft_expert_count`` routed experts per token.
    ``dspark``: a small draft model on its own engine - ``speculation.dspark.checkpoint_path`` when given, else (random-weight runs) the
    default 2-layer draft shape of the target's width.  Returns (None, 0) when the engine at hand cannot host the draft."""
    from ..speculation.model_draft import EngineDraft, draft_shape_for
    sp = cfg["speculation"]
    target = getattr(engine, "_engine", engine)                  # unwrap tracing / SPMD facades
    if sp["method"] == "mtp":
        # the model's own multi-token-prediction block, kept in step on the device: one proposed token per round
        from ..speculation.mtp_draft import DeviceMtpDraft, MtpDraft
        try:
            if hasattr(target, "enable_mtp"):
                return DeviceMtpDraft(target, sp["mtp"]), 1
            return MtpDraft(target, sp["mtp"]), (args.speculation_depth if args.speculation_depth is not None else sp["mtp"]["max_depth"])
        except (NotImplementedError, ValueError, AttributeError) as e:
            log.warning("MTP draft unavailable (%s); serving without speculation", e)
            return None, 0
    if sp["method"] == "self_speculative":
        from ..speculation.self_draft import SelfSpeculativeDraft
        depth = args.speculation_depth if args.speculation_depth is not None else sp["mtp"]["max_depth"]
        try:
            return SelfSpeculativeDraft(target, sp["self_speculative"], max_gamma=max(1, depth), layer_skip=sp.get("layer_skip_draft"),
                                        calibration=sp.get("calibration")), depth
        except (TypeError, NotImplementedError) as e:
            log.warning("self-speculative draft unavailable (%s); serving without speculation", e)
            return None, 0
    ds = sp["dspark"]
    depth = args.speculation_depth if args.speculation_depth is not None else ds["speculative_tokens"]
    block = build_block_draft(cfg, shape, target, args)
    if block is not None:
        return block, min(depth, block.max_tokens)
    if ds["checkpoint_path"]:
        from ..speculation.dspark import is_dspark_checkpoint
        if is_dspark_checkpoint(ds["checkpoint_path"]):
            return None, 0                                   # a block-draft checkpoint is no autoregressive draft model
    if args.test_engine:
        from ..runtime.null_engine import NullEngine
        return EngineDraft(NullEngine(vocab=target.vocab, max_seqs=2, max_ctx=target.max_ctx), max_gamma=depth), depth
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        log.warning("model draft with tensor-parallel serving is not wired; serving without speculation")
        return None, 0
    import torch
    from ..models.device_model import DeviceModel
    from ..runtime.engine import Engine
    dev = torch.device("cuda", int(ds["draft_gpus"][0]) if ds["draft_gpus"] else int(os.environ.get("LOCAL_RANK", 0)))
    page = cfg["memory"]["kv_cache"]["page_size_tokens"]
    if ds["checkpoint_path"]:
        from ..models.checkpoint import open_checkpoint
        dshape, w = open_checkpoint(ds["checkpoint_path"])
        dm = DeviceModel.from_state_dict(dshape, w, dev, "bf16", page)
    else:
        dshape = draft_shape_for(shape, quant="nvfp4" if ds["draft_weights_quant"] in ("nvfp4", "auto") else "bf16")
        log.warning("speculation.dspark.checkpoint_path is empty: RANDOM draft weights of shape %s", dshape.name)
        dm = DeviceModel.random_init(dshape, dev, "bf16", page)
    ctx = min(cfg["serving"]["max_sequence_length"], max(ds["draft_context_capacity_tokens"], 1024))
    # speculation.dspark.confidence_enabled: stop drafting at the first token the draft model itself gives less than
    # confidence_threshold (top-1 probability, computed on the device next to the token)
    min_conf = float(ds["confidence_threshold"]) if ds.get("confidence_enabled") else 0.0
    return EngineDraft(Engine(dm, max_seqs=2, max_ctx=ctx, prefill_chunk=cfg["orchestrator"]["prefill_chunk_tokens"], max_batch=1), max_gamma=depth,
                       min_confidence=min_conf), depth


def build_server(cfg: dict, shape: ModelConfig, ckpt: Optional[str], engine, args: argparse.Namespace):
    from ..serving.http_server import LayerStormServer, ServerConfig
    from ..serving.orchestrator import Orchestrator
    from ..serving.prefix_cache import PrefixCacheConfig
    from ..serving.tokenizer import TokenizerWrapper, resolve_tokenizer_dir
    sv = cfg["serving"]
    tpath = None if sv["tokenizer_mode"] == "byte" else resolve_tokenizer_dir(None if sv["tokenizer_path"] in ("", "auto") else sv["tokenizer_path"], ckpt)
    tok = TokenizerWrapper(tpath, vocab_limit=getattr(engine, "vocab", None) or shape.vocab)
    pc = sv["prefix_cache"]
    pcc = PrefixCacheConfig(enabled=pc["enabled"] and pc["max_entries"] > 0, max_tokens=pc["max_cached_tokens"], max_holders=max(1, pc["max_entries"]))
    pci = cfg.get("_internal-prefix_cache") or {}
    target = getattr(engine, "_engine", engine)
    if pcc.enabled and pci.get("hibernate_holders", False) and hasattr(target, "enable_kv_tiering") and int(os.environ.get("WORLD_SIZE", 1)) == 1:
        # idle prefix holders leave HBM for pinned host memory, and from there for files under the spill directory
        from ..serving.prefix_cache import PrefixSpillConfig
        page = cfg["memory"]["kv_cache"]["page_size_tokens"]
        try:
            target.enable_kv_tiering(int(pci.get("cold_pages", 0)) or max(64, pc["max_cached_tokens"] // page + pcc.max_holders))
            pcc.hibernate_holders = True
            pcc.hibernate_idle_seconds = float(pci.get("hibernate_idle_seconds", 30.0))
            pcc.spill = PrefixSpillConfig.from_config(cfg)
        except (NotImplementedError, RuntimeError) as e:
            log.warning("prefix holders stay in HBM: %s", e)
    eos = list(shape.eos_token_ids) or ([tok.eos_token_id] if getattr(tok, "eos_token_id", None) is not None else [])
    draft, depth = None, 0
    sp = cfg["speculation"]
    if sp["enabled"] and sp["method"] == "prompt_lookup":
        from ..speculation.prompt_lookup import PromptLookupDraft
        pl = sp["prompt_lookup"]
        draft = PromptLookupDraft(pl["min_ngram_size"], pl["max_ngram_size"], pl["max_continuation_length"])
        depth = args.speculation_depth if args.speculation_depth is not None else pl["max_continuation_length"]
    elif sp["enabled"] and sp["method"] in ("dspark", "self_speculative", "mtp"):
        draft, depth = build_model_draft(cfg, shape, engine, args)
        dcb, pl = sp["draft_combiner"], sp["prompt_lookup"]
        if draft is not None and dcb["enabled"] and pl["enabled"] and os.environ.get("LSB_DRAFT_COMBINER", "1") != "0":
            # the free source first: where the context repeats itself, prompt lookup proposes without running a model; otherwise the
            # model draft; the proposal with the most expected tokens per unit of cost goes to the target
            from ..speculation.combiner import DraftCombiner, DraftSource
            from ..speculation.prompt_lookup import IncrementalPromptLookup
            cost = {"dspark": dcb["dspark_compute_cost"], "mtp": dcb["mtp_compute_cost"], "self_speculative": dcb["self_spec_compute_cost"]}[sp["method"]]
            # (the indexed form: it is asked every round, and a rescan of a long context would cost more than a decode step)
            lookup = IncrementalPromptLookup(pl["min_ngram_size"], pl["max_ngram_size"], pl["max_continuation_length"])
            draft = DraftCombiner([DraftSource("prompt_lookup", lookup, cost=0.0, priority_boost=dcb["prompt_lookup_priority_boost"]),
                                   DraftSource(sp["method"], draft, cost=float(cost))])
    # continuous batching: as many plain greedy requests decode together as the engine's batched step takes (its CUDA graphs are
    # captured per batch size), bounded by the admitted concurrency
    eng_batch = int(getattr(getattr(engine, "_engine", engine), "max_batch", 1) or 1)
    # (LSB_SERVE_MAX_BATCH, default 8: every batch size that occurs gets its own step workspace and CUDA graph, which a model that
    # fills the GPU cannot afford for large batches)
    batch = max(1, min(eng_batch, int(cfg["orchestrator"]["max_batch_size"]), int(sv["max_concurrent_requests"]), int(os.environ.get("LSB_SERVE_MAX_BATCH", "8"))))
    policy = None
    if draft is not None and depth > 0 and os.environ.get("LSB_DEPTH_POLICY", "1") != "0":
        # speculation.utility_scorer / speculation.calibration: the depth asked of the draft follows the measured acceptance
        from ..speculation.combiner import DepthPolicy
        policy = DepthPolicy.from_config(sp, depth)
    reasoning = None
    if draft is not None and sp["reasoning_mode"]["enabled"]:
        # speculation.reasoning_mode: deeper drafts inside a think block; the block's markers come from serving.reasoning_config
        # ({"think_open": "...", "think_close": "..."}) or default to <think> ... </think>
        from ..speculation.policies import ReasoningMode
        marks = sv["reasoning_config"]
        marks = (json.load(open(marks)) if os.path.exists(marks) else json.loads(marks)) if marks else {}
        o, c = tok.encode(marks.get("think_open", "<think>")), tok.encode(marks.get("think_close", "</think>"))
        if o and c:
            reasoning = (ReasoningMode(sp["reasoning_mode"]), o, c)
    orch = Orchestrator(engine, eos_token_ids=eos, prefix_cache=pcc, draft=draft, speculation_depth=depth, tokenizer=tok, max_batch=batch, depth_policy=policy,
                        reasoning=reasoning,
                        prefill_slice_tokens=prefill_slice_factor(cfg) * int(cfg["orchestrator"]["prefill_chunk_tokens"]),
                        degraded_retry_max=int((cfg.get("_internal-orchestrator") or {}).get("degraded_retry_max", 1)
                                               if (cfg.get("_internal-orchestrator") or {}).get("degraded_retry_enabled", True) else 0))
    rc = sv["reasoning_config"]
    if rc:
        rc = json.load(open(rc)) if os.path.exists(rc) else json.loads(rc)
    scfg = ServerConfig(model_name=sv["model_name"] or shape.name, max_concurrent=sv["max_concurrent_requests"],
                        max_queued_requests=sv["max_queued_requests"], sse_heartbeat_seconds=sv["sse_heartbeat_seconds"],
                        max_sequence_length=sv["max_sequence_length"], tool_call_parser=sv["tool_call_parser"] or None,
                        enable_auto_tool_choice=sv["enable_auto_tool_choice"], reasoning_parser=sv["reasoning_parser"] or None,
                        reasoning_config=rc or None)
    return LayerStormServer(orch, tok, scfg), orch


def start_rank_liveness(world: int):
    """Heartbeats of every rank through the job's rendezvous store; on rank 0 also the monitor that SpmdLeader asks before each step
    (LS_RANK_TIMEOUT_S, default 10 s; 0 disables).  Returns (monitor or None, heartbeat or None)."""
    timeout = float(os.environ.get("LS_RANK_TIMEOUT_S", "10"))
    if timeout <= 0:
        return None, None
    try:
        import torch.distributed as dist
        from torch.distributed.distributed_c10d import _get_default_store
        store = dist.PrefixStore("lsb200_hb", _get_default_store())
    except Exception as e:            # noqa: BLE001 - liveness is an extra; serving works without it
        log.warning("rank liveness disabled: no rendezvous store (%s)", e)
        return None, None
    from ..runtime.heartbeat import Heartbeat, RankMonitor
    rank = int(os.environ.get("RANK", 0))
    beat = Heartbeat(store, rank, interval_s=min(1.0, timeout / 5)).start()
    monitor = RankMonitor(store, list(range(1, world)), timeout_s=timeout).start(interval_s=min(1.0, timeout / 5)) if rank == 0 else None
    return monitor, beat


def apply_live_changes(changes, orch, cfg: Optional[dict] = None) -> None:
    """Push hot-reloaded fields into the running components.  The config tree itself is already updated in place."""
    evict = False
    for path, old, new in changes:
        log.info("config hot reload: %s %r -> %r", path, old, new)
        if path == "speculation.mtp.max_depth" and getattr(orch, "draft", None) is not None:
            orch.gamma = max(0, int(new))
        evict |= path.startswith("memory.expert_cache.eviction_")
    engine = getattr(orch, "engine", None)
    if evict and cfg is not None and hasattr(engine, "configure_expert_cache"):
        engine.configure_expert_cache(cfg["memory"]["expert_cache"])      # through the SPMD facade: every rank's cache takes it


def main(argv: Optional[list[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    logging.basicConfig(level=getattr(logging, args.log_level.upper()), format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    os.environ.setdefault("CUDA_DEVICE_ORDER", "PCI_BUS_ID")
    try:
        cfg, shape, ckpt, explain = resolve_config(args)
    except ConfigError as e:
        print(str(e), file=sys.stderr)
        return 2
    except Exception as e:
        from ..autoconfig import AutoconfigRefusal
        if isinstance(e, AutoconfigRefusal):
            print(f"autoconfig refused: {e}\n  relax: {e.binding}", file=sys.stderr)
            return 3
        raise
    if explain:
        log.info("%s", explain)
    if args.dry_run:
        print(json.dumps(cfg, indent=1))
        return 0
    engine = build_engine(cfg, shape, ckpt, args)
    world = int(os.environ.get("WORLD_SIZE", 1)) if not args.test_engine else 1
    monitor = None
    if world > 1:
        # SPMD: rank 0 runs the orchestrator and the HTTP server and announces every engine call; the other ranks replay them
        from ..runtime.spmd import SpmdLeader, control_group, follower_loop
        grp = control_group()
        monitor, beat = start_rank_liveness(world)
        if int(os.environ.get("RANK", 0)) != 0:
            # an engine call that fails (e.g. KV pool exhausted) fails the same way on every rank; the leader's orchestrator handles
            # it (evict / retry / degrade), the followers just log it and wait for the next call
            follower_loop(engine, grp, on_error=lambda name, e: log.warning("replayed %s raised %s: %s", name, type(e).__name__, e))
            if beat is not None:
                beat.stop(goodbye=True)
            return 0
        engine = SpmdLeader(engine, grp, monitor=monitor)
    tracer = None
    from ..utils import perf_trace
    if perf_trace.enabled():
        # LS_PERF_TRACE: begin / end records around every engine call, dumped with a report at shutdown
        tracer = perf_trace.Tracer(gpu=int(os.environ.get("LOCAL_RANK", 0)))
        engine = perf_trace.TracedEngine(engine, tracer)
    server, orch = build_server(cfg, shape, ckpt, engine, args)
    if world > 1 and monitor is not None:
        server.failed_ranks = lambda: dict(monitor.failed)       # /health answers 503 while a rank is down
    reloader = None
    if args.config and not args.autoconfig:
        # hot reload of the live-changeable fields; everything else in an edited file is reported and waits for a restart
        from ..config.hot_reload import ConfigHotReloader
        reloader = ConfigHotReloader(args.config, cfg, overrides_from_args(args), on_apply=lambda ch: apply_live_changes(ch, orch, cfg))
        reloader.start()
    idle = (args.cycle_budget_us or 200) * 1e-6
    t = threading.Thread(target=orch.run, kwargs={"idle_sleep_s": idle}, name="orchestrator", daemon=True)
    t.start()
    try:
        server.run(cfg["serving"]["host"], cfg["serving"]["port"], args.log_level)
    finally:
        if reloader is not None:
            reloader.stop()
        orch.shutdown()
        t.join(timeout=5)
        if world > 1:
            engine.shutdown()
        if tracer is not None:
            rep = tracer.dump(perf_trace.out_path())
            log.info("perf trace: %d records -> %s\n%s", rep["records"], perf_trace.out_path(), perf_trace.format_table(rep))
    return 0


if __name__ == "__main__":
    sys.exit(main())
