"""`cuteafd` command line: serve | plan | golden | expertd | fabric | bench | doctor.

    python -m cuteafd_b200.cli plan qwen3-235b --layout
    python -m cuteafd_b200.cli serve --model tiny --listen 127.0.0.1:8000
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m cuteafd_b200.cli serve --model deepseek-v3
        (attention TP2 on ranks 0-1 + experts on ranks 2-7; rank 0 runs the scheduler and the HTTP server, see serving/split.py)

`serve` auto-detects the family from a snapshot's config.json (or takes a named synthetic shape), sizes the KV pool
with the placement solver, builds the engine, and starts the HTTP server once the scheduler thread is ready.
Reference: cuteafd-daemon/src/cli.rs:44-115 (commands), :857-1005 (serve flags), commands/plan.rs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def cmd_plan(a) -> int:
    from .loader.plan import plan
    rep = plan(a.model, world=a.gpus, layout=a.layout or a.deployment, files=a.files, pool_tokens=a.pool_tokens, gpu_gib=a.gpu_gib, stages=a.stages,
               attn_groups=a.attn_groups)
    if a.rank >= 0 and os.path.isdir(a.model):
        from .config import default_deployment
        from .loader.plan import files_for_rank
        n_exp = rep.spec.moe.n_experts if rep.spec is not None else None
        print(json.dumps(files_for_rank(a.model, default_deployment(a.gpus, a.attn_groups), a.rank, n_exp), indent=2))
        return 0
    if a.deployment and rep.layout is not None:
        from .loader.plan import deployment_decisions
        print(json.dumps(deployment_decisions(rep.layout, a.model), indent=2))
        return 0 if rep.supported else 2
    print(json.dumps(rep.to_json(), indent=2) if a.json else rep.text())
    return 0 if rep.supported else 2


def cmd_doctor(a) -> int:
    import torch
    from .ops import native
    info = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "native_library": str(native.LIB_PATH),
            "native_library_present": native.available()}
    if native.available():
        try:
            info["abi_version"] = native.lib().cuteafd_abi_version()
        except Exception as e:
            info["native_error"] = str(e)
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        info.update(gpu=p.name, sms=p.multi_processor_count, memory_gib=round(p.total_memory / 2 ** 30, 1),
                    compute_capability=f"{p.major}.{p.minor}", n_gpus=torch.cuda.device_count())
        info["p2p"] = [[torch.cuda.can_device_access_peer(i, j) if i != j else True for j in range(torch.cuda.device_count())]
                       for i in range(torch.cuda.device_count())]
    print(json.dumps(info, indent=2))
    return 0


def cmd_fabric(a) -> int:
    """NVLink link probes (copy engine vs SM push vs SM pull, one-way vs duplex, eager vs graph, flag round trip, all-to-all):
    `python -m torch.distributed.run --nproc-per-node N -m cuteafd_b200.cli fabric [--all-to-all]`.  Reference: `cuteafd fabric --p2p`."""
    if int(os.environ.get("WORLD_SIZE", "1")) < 2:
        print(json.dumps({"error": "the fabric probe runs one rank per GPU: python -m torch.distributed.run --nproc-per-node 2 "
                                   "--master-addr 127.0.0.1 -m cuteafd_b200.cli fabric"}))
        return 2
    from .bench import fabric
    sys.argv = ["fabric"] + (["--all-to-all"] if a.all_to_all else []) + (["--sizes", a.sizes] if a.sizes else [])
    return fabric.main()


def build_serving(a):
    """Engine + scheduler + prefix cache for a model name or snapshot.  One process: a single-GPU engine.  Under torchrun
    (WORLD_SIZE > 1): the attention/expert split; only the leader gets a scheduler back, the other ranks serve inside this call
    and it returns None for them when the leader stops."""
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        from .serving.split import build_split_serving
        return build_split_serving(a, world)
    from .config import spec_from_snapshot, spec_by_name, NAMED_SPECS, QuantSpec
    from .engine.engine import Engine
    from .engine.kv import PagePool
    from .models.weights import DeviceWeights
    from .ref.model import init_weights
    from .serving.prefix import PrefixCache
    from .serving.runner import EngineRunner, attach_pool
    from .serving.scheduler import NgramDrafter, Scheduler
    spec = spec_by_name(a.model) if a.model in NAMED_SPECS else spec_from_snapshot(a.model)
    dev = torch.device("cuda", a.device)
    layers = getattr(a, "layers", 0)
    if layers:
        spec = spec.replace(n_layers=layers)
    if os.path.isdir(a.model) and spec.attn.kind == "gqa":
        from .loader.checkpoint import load_device_weights
        weights = load_device_weights(a.model, spec, dev)      # tensors in their stored formats, no repacking
    elif spec.name == "tiny":
        weights = DeviceWeights.from_masters(spec, init_weights(spec, 0), dev)
    else:
        weights = DeviceWeights.random(spec, dev, seed=1)      # named shapes without a snapshot: synthetic weights
    n_pages = a.pool_tokens // 64 if a.pool_tokens else 4096
    if getattr(a, "gpu_occupancy_percent", 0):
        # pool sized by the start-up capacity policy from the memory measured now (the weights are already resident); a pool that was
        # asked for and does not fit is an error, only the default pool is sized down
        from .serving.capacity import CapacityPolicy, plan_capacity
        free, total = torch.cuda.mem_get_info(dev)
        cap = plan_capacity(CapacityPolicy(concurrency=a.max_sequences, target_pool_tokens=a.pool_tokens, gpu_occupancy_percent=a.gpu_occupancy_percent),
                            total_bytes=total, free_bytes=free, weight_bytes=weights.nbytes(), kv_bytes_per_token=spec.kv_bytes_per_token(),
                            model_max_context=spec.max_context, weights_loaded=True)
        print(f"[serve] capacity: {cap.describe()}", file=sys.stderr)
        n_pages = cap.pool_pages
    eng = Engine(weights, n_pages=n_pages, max_seqs=a.max_sequences, max_pages_per_seq=min(n_pages, a.max_context // 64 + 1))
    pool = PagePool(n_pages)
    runner = attach_pool(EngineRunner(eng, max_rows=a.prefill_batch_tokens), pool)
    host = None
    if getattr(a, "host_cache_gib", 0) > 0:
        from .serving.hostcache import attach_host_tier
        host = attach_host_tier(eng, max(0.0, a.host_cache_gib - a.host_cache_headroom_gib), min_tokens=a.host_cache_min_tokens)
    prefix = PrefixCache(pool, max_entries=a.prefix_cache_entries, min_tokens=a.prefix_cache_min_tokens, host=host)
    recurrent = bool(spec.attn.linear_every)
    if recurrent:
        # gated delta-rule layers carry a recurrent state per sequence: a request cannot resume from cached pages (drafted steps are
        # fine: they leave the state alone and the accepted rows are replayed into it)
        prefix = None
        print(f"[serve] {spec.name}: linear-attention layers - the prefix cache is off", file=sys.stderr)
    drafter = None
    if a.draft == "ngram":
        drafter = NgramDrafter()
    elif a.draft == "mtp" and not recurrent:
        from .serving.mtp_drafter import MtpDrafter
        drafter = MtpDrafter(runner)                           # the model's own MTP module (needs MTP weights)
    policy = None
    if getattr(a, "draft_policy", "simple") == "online" and drafter is not None:
        from .serving.draft_policy import OnlineDraftPolicy
        m = spec.moe
        # bytes of one routed expert (gate + up + down) in its stored format, as the price unit of the traffic forecast
        per_weight = {"bf16": 2.0, "fp8_block128": 1.0}.get(spec.quant.experts, 0.5625)
        policy = OnlineDraftPolicy(max(a.draft_limit, 1), n_experts=m.n_experts, top_k=m.top_k,
                                   slice_mb=3 * spec.hidden * m.intermediate * per_weight / 2 ** 20)
    sched = Scheduler(runner, pool, max_seqs=a.max_sequences, prefill_chunk=a.prefill_batch_tokens, decode_share=a.decode_share,
                      prefix=prefix, drafter=drafter, max_draft=a.draft_limit, queue_limit=getattr(a, "http_queue", 64),
                      queue_wait_s=getattr(a, "queue_wait_s", 0) or None, policy=policy)
    return spec, sched


def _aliases(a) -> dict:
    """`--official-model-names a,b,c` and/or `--official-model-names-file FILE` (one name per line)."""
    names = [n for n in (a.official_model_names or "").split(",") if n]
    if a.official_model_names_file:
        names += [l.strip() for l in open(a.official_model_names_file) if l.strip() and not l.startswith("#")]
    return {n: "served" for n in names}


def _search_provider(a):
    """--search-corpus FILE (JSON list of {title, url, text}) | --searxng URL | --exa-key-file FILE; none = no search endpoint."""
    from .serving.gateway_extras import CorpusProvider, ExaProvider, SearxngProvider
    if getattr(a, "search_corpus", ""):
        return CorpusProvider(json.load(open(a.search_corpus)))
    if getattr(a, "searxng", ""):
        return SearxngProvider(a.searxng)
    if getattr(a, "exa_key_file", ""):
        return ExaProvider(open(a.exa_key_file).read().strip())
    return None


def _gateway_args(p):
    p.add_argument("--record", default="", help="append every POST request / response pair to this JSONL file")
    p.add_argument("--search-corpus", default="", help="JSON file of documents served by /v1/alpha/search (offline provider)")
    p.add_argument("--searxng", default="", help="base URL of a SearXNG instance for /v1/alpha/search")
    p.add_argument("--exa-key-file", default="", help="file holding an Exa API key for /v1/alpha/search")


def cmd_gateway(a) -> int:
    """The gateway surfaces (Anthropic Messages, OpenAI Responses, aliases, CORS) over a CPU stand-in model: lets
    client integrations be developed without a GPU.  With a GPU the same surfaces are part of `serve --gateway on`.
    Reference: cuteafd-daemon/src/commands/gateway.rs."""
    from .engine.kv import PagePool
    from .serving.api import ServingLoop, build_app
    from .serving.chat_templates import template_for
    from .serving.runner import FakeRunner
    from .serving.scheduler import Scheduler
    runner = FakeRunner(vocab=258)
    runner.next_token = lambda prefix: 257 if len(prefix) % 97 == 0 else 32 + (sum(prefix[-3:]) % 90)
    loop = ServingLoop(Scheduler(runner, PagePool(1024))).start()
    app = build_app(loop, model_id=a.model_id, template=template_for(a.chat_template or "plain"), model_aliases=_aliases(a),
                    allow_origin=a.gateway_allow_origin or None, enable_bench=True, search=_search_provider(a), record_path=a.record or None)
    if a.replay:                 # play a recorded session back against the stand-in model (or --replay-url) and report differences
        from .serving.gateway_extras import replay
        rep = replay(a.replay_url or app, a.replay)
        print(json.dumps(rep))
        loop.stop()
        return 0 if not rep["mismatches"] else 1
    host, port = a.listen.rsplit(":", 1)
    import uvicorn
    uvicorn.run(app, host=host, port=int(port), log_level="info")
    return 0


def cmd_serve(a) -> int:
    from .loader.tokenizer import load_tokenizer
    from .serving.api import ServingLoop, build_app
    from .serving.chat_templates import template_for
    built = build_serving(a)
    if built is None:            # a follower or expert rank of a multi-GPU layout: it has served and is done
        return 0
    spec, sched = built
    loop = ServingLoop(sched).start()
    keys = set(open(a.api_key_file).read().split()) if a.api_key_file else None
    usage = thermal = None
    if a.usage == "on":
        from .serving.usage import UsageStore
        os.makedirs(a.usage_dir, exist_ok=True)
        usage = UsageStore(os.path.join(a.usage_dir, "usage.sqlite"))
    try:
        from .utils.thermal import ThermalMonitor
        thermal = ThermalMonitor().start()          # background sampler behind the window summaries of /v1/thermal (reads only)
    except Exception:
        thermal = None
    vision = _vision_front_end(a, spec)
    app = build_app(loop, model_id=a.model_id or spec.name, tokenizer=load_tokenizer(a.model if os.path.isdir(a.model) else None), vision=vision,
                    api_keys=keys, max_output=a.max_output, template=template_for(a.chat_template or spec.name),
                    usage=usage, enable_bench=a.enable_bench, thermal=thermal, gateway=a.gateway == "on",
                    model_aliases=_aliases(a), allow_origin=a.gateway_allow_origin or None, search=_search_provider(a),
                    record_path=a.record or None)
    host, port = a.listen.rsplit(":", 1)
    import uvicorn
    uvicorn.run(app, host=host, port=int(port), log_level="info")
    return 0


def _vision_front_end(a, spec):
    """The vision tower of `serve`: `--vision auto` builds it when the snapshot has a `vision_config` and `visual.*` tensors, `--vision
    random:DEPTH` builds a randomly initialised tower of the Qwen-VL shape for shape / throughput work, `--vision off` (and multi-GPU
    layouts, whose engines take token ids only) serve text alone.  Reference: cuteafd-daemon/src/cli.rs (vision / audio encoder flags)."""
    mode = getattr(a, "vision", "auto")
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return None
    import torch
    from .models.vision import VisionTower
    from .serving.vision import VisionFrontEnd
    dev = torch.device("cuda", a.device)
    audio_kw = {}
    amode = getattr(a, "audio", "off")
    if amode.startswith("random"):          # a randomly initialised encoder of the Whisper-large shape (32 blocks by default)
        from .models.audio import AudioTower
        from .ref.audio import AudioSpec, init_audio_weights
        depth = int(amode.split(":", 1)[1]) if ":" in amode else 2
        asp = AudioSpec(hidden=1280, depth=depth, n_heads=20, head_dim=64, intermediate=5120, out_hidden=spec.hidden, n_mels=128)
        audio_kw = dict(audio_tower=AudioTower(asp, init_audio_weights(asp, 0), dev), audio_pad_id=min(spec.vocab - 2, 151646))
    if mode.startswith("random"):
        from .ref.vision import VisionSpec, init_vision_weights
        depth = int(mode.split(":", 1)[1]) if ":" in mode else 2
        vs = VisionSpec(hidden=1152, depth=depth, n_heads=16, head_dim=72, intermediate=4304, patch=16, out_hidden=spec.hidden, pos_grid=48)
        tower = VisionTower(vs, init_vision_weights(vs, 0), dev, max_patches=a.vision_max_patches)
        return VisionFrontEnd(tower, pad_id=min(spec.vocab - 1, 151655), start_id=None, end_id=None, max_images=a.vision_max_images, **audio_kw)
    if mode == "off" or not os.path.isdir(a.model):
        return VisionFrontEnd(None, max_images=a.vision_max_images, **audio_kw) if audio_kw else None
    from .loader.vision_checkpoint import read_vision_masters, vision_spec_from_snapshot
    found = vision_spec_from_snapshot(a.model)
    if found is None:
        return VisionFrontEnd(None, max_images=a.vision_max_images, **audio_kw) if audio_kw else None
    vs, ids = found
    if vs.out_hidden != spec.hidden:
        raise SystemExit(f"vision tower emits rows of {vs.out_hidden}, the decoder's hidden size is {spec.hidden}")
    tower = VisionTower(vs, read_vision_masters(a.model, vs), dev, max_patches=a.vision_max_patches)
    print(f"vision tower: depth {vs.depth}, hidden {vs.hidden}, {tower.nbytes() / 2**20:.0f} MiB", flush=True)
    return VisionFrontEnd(tower, pad_id=int(ids["pad"]), start_id=ids["start"], end_id=ids["end"], max_images=a.vision_max_images, **audio_kw)


def cmd_bench_history(a) -> int:
    """`bench-history add [FILE|-] | list | compare A B | regressions | report [--svg OUT] | matrix`: the SQLite history of measured
    benchmark lines (reference: cuteafd-bench history / reports / release smoke matrix)."""
    import json
    import sys
    from .bench.history import BenchHistory, smoke_matrix
    if a.action == "matrix":
        for row in smoke_matrix():
            print(f"{row['name']:<34} {row['cmd']}")
        return 0
    os.makedirs(os.path.dirname(os.path.abspath(a.db)), exist_ok=True)
    h = BenchHistory(a.db)
    if a.action == "add":
        src = sys.stdin if not a.args or a.args[0] == "-" else open(a.args[0])
        n = 0
        for text in src:
            text = text.strip()
            if text.startswith("{"):
                try:
                    line = json.loads(text)
                except ValueError:
                    continue
                if "metric" in line and "value" in line:
                    print(f"run {h.add(line, label=a.label, commit_id=a.commit)}: {line['metric']} = {line['value']} {line.get('unit', '')}")
                    n += 1
        return 0 if n else 1
    if a.action == "list":
        print(h.report_markdown(a.metric or None))
    elif a.action == "compare":
        print(json.dumps(h.compare(int(a.args[0]), int(a.args[1]), a.tolerance), indent=1))
    elif a.action == "regressions":
        regs = h.latest_regressions(a.tolerance)
        print(json.dumps(regs, indent=1))
        return 1 if regs else 0
    elif a.action == "report":
        print(h.report_markdown(a.metric or None))
        if a.svg:
            open(a.svg, "w").write(h.report_svg(a.metric or "decode_tokens_per_s"))
            print(f"trend -> {a.svg}")
    return 0


def cmd_usage(a) -> int:
    """`usage clear | clear-log | export-csv | demo`: manage the request history without a browser; `demo` serves
    `/usage` over a synthetic history (no GPU, no model).  Reference: cuteafd-daemon/src/commands/usage.rs."""
    import sys
    from .serving.usage import UsageStore, synthetic_history
    path = os.path.join(a.dir, "usage.sqlite") if a.dir != ":memory:" else ":memory:"
    if a.action == "demo":
        from .engine.kv import PagePool
        from .serving.api import ServingLoop, build_app
        from .serving.runner import FakeRunner
        from .serving.scheduler import Scheduler
        store = UsageStore(":memory:")
        synthetic_history(store)
        loop = ServingLoop(Scheduler(FakeRunner(vocab=258), PagePool(256))).start()
        app = build_app(loop, model_id="demo-model", usage=store)
        host, port = a.listen.rsplit(":", 1)
        import uvicorn
        uvicorn.run(app, host=host, port=int(port), log_level="info")
        return 0
    os.makedirs(a.dir, exist_ok=True)
    store = UsageStore(path)
    if a.action == "clear":
        store.clear()
    elif a.action == "clear-log":
        store.clear_log()
    elif a.action == "export-csv":
        out = open(a.out, "w", newline="") if a.out else sys.stdout
        n = store.export_csv(out, a.range)
        if a.out:
            out.close()
            print(f"{n} rows -> {a.out}")
    return 0


def _golden_masters(model: str):
    """(spec, fp32 masters) of a model the CPU oracle can evaluate: the tiny model or a snapshot directory."""
    import os
    from .config import spec_from_snapshot, tiny_spec
    from .ref.model import init_weights
    if model == "tiny":
        spec = tiny_spec()
        return spec, init_weights(spec, 0)
    if not os.path.isdir(model):
        raise SystemExit(f"golden windows need fp32 masters: give the tiny model or a snapshot directory, not {model!r}")
    from .loader.checkpoint import read_masters
    spec = spec_from_snapshot(model)
    return spec, read_masters(model, spec)


def cmd_golden(a) -> int:
    """`golden --write FILE [--model M]`: seal golden windows from the fp32 oracle.  `golden --check FILE [--model M]`: check the GPU
    engine's logits against a golden file.  Without either: teacher-forced comparison of the tiny model against the oracle."""
    import torch
    if getattr(a, "write", None):
        from .bench.golden import write_golden
        spec, masters = _golden_masters(a.model)
        gold = write_golden(a.write, spec, masters, n=a.windows, length=a.window_tokens, seed=a.seed or 2026)
        print(json.dumps({"wrote": a.write, "model": gold["model"], "digest": gold["digest"], "windows": len(gold["windows"])}))
        return 0
    if getattr(a, "check", None):
        from .bench.golden import check_logits, engine_logits_fn, read_golden
        import argparse
        ns = argparse.Namespace(model=a.model, device=0, max_context=4096, max_sequences=4, pool_tokens=0, prefill_batch_tokens=4096, decode_share=0.2,
                                prefix_cache_entries=4, prefix_cache_min_tokens=64, draft="off", draft_limit=0, layers=0, host_cache_gib=0.0)
        spec, sched = build_serving(ns)
        rep = check_logits(engine_logits_fn(sched.runner.eng), read_golden(a.check), spec=spec)
        print(json.dumps(rep))
        return 0 if rep["pass"] else 1
    from .config import tiny_spec, QuantSpec
    from .engine.engine import Engine
    from .engine.generate import BatchGenerator
    from .models.weights import DeviceWeights
    from .ref.model import RefCache, RefModel, init_weights
    spec = tiny_spec().replace(quant=QuantSpec(experts=a.experts, dense="bf16"))
    dw = DeviceWeights.from_masters(spec, init_weights(spec, a.seed), "cuda")
    eng = Engine(dw, n_pages=32, max_seqs=8, max_pages_per_seq=4)
    ref = RefModel(spec, dw.dequantized_masters())
    g = torch.Generator().manual_seed(a.seed)
    prompts = [torch.randint(0, spec.vocab, (64,), generator=g).tolist() for _ in range(2)]
    gen = BatchGenerator(eng)
    gen.prefill(prompts)
    lane = eng.lane(128)
    out = []
    for i, p in enumerate(prompts):
        rl, _ = ref.forward(torch.tensor(p), 0, RefCache())
        got = lane.logits[i].float().cpu()
        out.append({"prompt": i, "rel_l2": float((got - rl[-1]).norm() / rl[-1].norm()), "top1_match": int(got.argmax()) == int(rl[-1].argmax())})
    print(json.dumps({"family": "tiny", "experts": a.experts, "rows": out}))
    return 0 if all(r["rel_l2"] < 0.25 for r in out) else 1


def cmd_expertd(a) -> int:
    """Host-path expert service: answers framed expert waves over TCP with the synthetic executor (protocol bring-up
    and multi-host tests); the in-node data path uses peer memory and needs no daemon."""
    from .parallel.transport import ExpertServer, SyntheticRouteExecutor
    host, port = a.listen.rsplit(":", 1)
    srv = ExpertServer(SyntheticRouteExecutor(executor_id=a.rank), host, int(port))
    print(json.dumps({"listening": list(srv.address), "rank": a.rank}), flush=True)
    try:
        srv.thread.join()
    except KeyboardInterrupt:
        srv.stop()
    return 0


def cmd_card(a) -> int:
    """Baseline card (C1 decode, C4/C8/C16 aggregate, 8k prefill + TTFT, quick quality gates) through the scheduler."""
    import json
    import torch
    from .bench.card import run_card
    state = {}

    def make():
        # one engine for the whole card (weights stay resident); every section gets a fresh scheduler, pool and prefix cache
        if "eng" not in state:
            state["spec"], sched = build_serving(a)
            state["eng"] = sched.runner.eng
            return sched
        from .engine.kv import PagePool
        from .serving.prefix import PrefixCache
        from .serving.runner import EngineRunner, attach_pool
        from .serving.scheduler import NgramDrafter, Scheduler
        eng = state["eng"]
        pool = PagePool(eng.n_pages)
        runner = attach_pool(EngineRunner(eng, max_rows=a.prefill_batch_tokens), pool)
        return Scheduler(runner, pool, max_seqs=a.max_sequences, prefill_chunk=a.prefill_batch_tokens, decode_share=a.decode_share,
                         prefix=PrefixCache(pool, max_entries=a.prefix_cache_entries, min_tokens=a.prefix_cache_min_tokens),
                         drafter=NgramDrafter() if a.draft == "ngram" else None, max_draft=a.draft_limit)
    first = make()                                             # builds the engine; its spec gives the vocabulary
    pending = [first]
    card = run_card(lambda: pending.pop() if pending else make(), vocab=state["spec"].vocab, c1_tokens=a.c1_tokens,
                    prefill_tokens=a.prefill_tokens)
    card["model"] = state["spec"].name
    card["layers"] = state["spec"].n_layers
    if getattr(a, "golden", None):          # logit fidelity against sealed golden windows (`cuteafd golden --write`)
        from .bench.golden import check_logits, engine_logits_fn, read_golden
        rep = check_logits(engine_logits_fn(state["eng"]), read_golden(a.golden), spec=state["spec"])
        card["quality"]["logit_fidelity"] = rep["pass"]
        card["quality"]["logit_fidelity_windows"] = rep["windows"]
    from .serving.chat_templates import template_round_trip
    card["quality"]["template_round_trip"] = template_round_trip(state["spec"].family)
    torch.cuda.synchronize()
    print(json.dumps(card))
    return 0


def cmd_run(a) -> int:
    """`run --config FILE [--set K=V ...] [--print]`: the operator's KEY=VALUE file becomes a command line."""
    import shlex
    from . import configfile
    try:
        argv = configfile.to_argv(configfile.load(a.config, a.set), a.subparsers)
    except configfile.ConfigError as e:
        print(f"config error: {e}", file=sys.stderr)
        return 2
    if a.print or a.dry_run:
        print("cuteafd " + " ".join(shlex.quote(x) for x in argv))
        return 0
    if a.restart and a.pidfile:
        _stop_pidfile(a.pidfile, a.stop_timeout)
    if a.detach:
        return _spawn_detached(argv, a.pidfile, a.log)
    return main(argv)


def _spawn_detached(argv: list, pidfile: str, log: str) -> int:
    """Start `cuteafd <argv>` as its own session (process group) with output in `log`, record its pid."""
    import subprocess
    if not pidfile:
        print("--detach needs --pidfile", file=sys.stderr)
        return 2
    if _pid_alive(_read_pid(pidfile)):
        print(f"already running (pid {_read_pid(pidfile)}; use --restart)", file=sys.stderr)
        return 1
    out = open(log or os.devnull, "ab")
    proc = subprocess.Popen([sys.executable, "-m", "cuteafd_b200.cli", *argv], stdout=out, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL,
                            start_new_session=True)
    os.makedirs(os.path.dirname(os.path.abspath(pidfile)), exist_ok=True)
    with open(pidfile, "w") as f:
        f.write(str(proc.pid))
    print(f"started pid {proc.pid}" + (f", log {log}" if log else ""))
    return 0


def _read_pid(pidfile: str) -> int | None:
    try:
        return int(open(pidfile).read().strip())
    except (OSError, ValueError):
        return None


def _pid_alive(pid: int | None) -> bool:
    if not pid:
        return False
    try:
        os.kill(pid, 0)
    except OSError:
        return False
    try:                                    # a finished child that nobody has waited for still has a pid
        return open(f"/proc/{pid}/stat").read().split(")")[-1].split()[0] != "Z"
    except OSError:
        return True


def _stop_pidfile(pidfile: str, timeout_s: float = 20.0) -> str:
    """Ends exactly the process group recorded in the pid file: SIGTERM, then SIGKILL when it has not gone after `timeout_s`."""
    import signal
    import time
    pid = _read_pid(pidfile)
    if not _pid_alive(pid):
        if pid is not None:
            os.unlink(pidfile)
        return "not running"
    for sig, wait in ((signal.SIGTERM, timeout_s), (signal.SIGKILL, 5.0)):
        try:
            os.killpg(pid, sig)             # the server was started as the leader of its own session
        except OSError:
            try:
                os.kill(pid, sig)
            except OSError:
                break
        t0 = time.time()
        while time.time() - t0 < wait:
            try:
                os.waitpid(pid, os.WNOHANG)         # reaps it when it is our child; otherwise the poll below sees it go
            except OSError:
                pass
            if not _pid_alive(pid):
                os.unlink(pidfile)
                return "stopped" if sig == signal.SIGTERM else "killed"
            time.sleep(0.05)
    return "still running"


def cmd_stop(a) -> int:
    """`stop --pidfile FILE`: end the server that `run --detach --pidfile FILE` started (reference: stop.sh beside run.sh)."""
    res = _stop_pidfile(a.pidfile, a.timeout)
    print(res)
    return 0 if res in ("stopped", "killed", "not running") else 1


def cmd_quantize(a) -> int:
    """`quantize SRC DST --dense FMT --experts FMT`: resumable re-quantisation of a snapshot (run the same command again
    after an interruption)."""
    from .config import spec_from_snapshot
    from .loader.quantize import quantize_snapshot
    spec = spec_from_snapshot(a.src)
    try:
        r = quantize_snapshot(a.src, a.dst, spec, dense=a.dense, experts=a.experts, restart=a.restart, log=lambda m: print(m, flush=True))
    except ValueError as e:
        print(f"quantize: {e}", file=sys.stderr)
        return 2
    print(json.dumps({"written": len(r["written"]), "skipped": len(r["skipped"]), "published": r["published"]}))
    return 0


def cmd_bench(a) -> int:
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return subprocess.call([sys.executable, os.path.join(root, "bench.py"), *a.rest])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="cuteafd")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("plan"); p.add_argument("model"); p.add_argument("--layout", action="store_true"); p.add_argument("--files", action="store_true")
    p.add_argument("--gpus", type=int, default=8); p.add_argument("--pool-tokens", type=int, default=0); p.add_argument("--gpu-gib", type=int, default=180)
    p.add_argument("--attn-groups", type=int, default=1, help="data-parallel attention groups sharing the expert ranks")
    p.add_argument("--deployment", action="store_true", help="print the typed launch decisions of the layout as JSON")
    p.add_argument("--rank", type=int, default=-1, help="with a snapshot directory: list the files and bytes this rank of the layout reads")
    p.add_argument("--stages", type=int, default=0, help="plan a layer-range split over this many GPUs (consecutive layer ranges, hidden-state hops)")
    p.add_argument("--json", action="store_true"); p.set_defaults(fn=cmd_plan)
    p = sub.add_parser("doctor"); p.set_defaults(fn=cmd_doctor)
    p = sub.add_parser("run"); p.add_argument("--config", required=True); p.add_argument("--set", action="append", default=[])
    p.add_argument("--print", action="store_true"); p.add_argument("--dry-run", action="store_true", help="same as --print")
    p.add_argument("--detach", action="store_true", help="start in the background as its own process group (needs --pidfile)")
    p.add_argument("--pidfile", default=""); p.add_argument("--log", default=""); p.add_argument("--restart", action="store_true",
                                                                                                   help="stop what the pid file names first")
    p.add_argument("--stop-timeout", type=float, default=20.0); p.set_defaults(fn=cmd_run, subparsers=sub.choices)
    p = sub.add_parser("stop"); p.add_argument("--pidfile", required=True); p.add_argument("--timeout", type=float, default=20.0)
    p.set_defaults(fn=cmd_stop)
    p = sub.add_parser("fabric"); p.add_argument("--p2p", action="store_true"); p.add_argument("--all-to-all", action="store_true")
    p.add_argument("--sizes", default="", help="comma-separated message sizes in bytes"); p.set_defaults(fn=cmd_fabric)
    p = sub.add_parser("bench-history"); p.add_argument("action", choices=["add", "list", "compare", "regressions", "report", "matrix"])
    p.add_argument("args", nargs="*"); p.add_argument("--db", default=os.path.expanduser("~/.cache/cuteafd-b200/bench/history.sqlite"))
    p.add_argument("--label", default=""); p.add_argument("--commit", default=""); p.add_argument("--metric", default="")
    p.add_argument("--tolerance", type=float, default=0.02); p.add_argument("--svg", default=""); p.set_defaults(fn=cmd_bench_history)
    p = sub.add_parser("serve")
    p.add_argument("--model", "--snapshot", dest="model", default="tiny"); p.add_argument("--listen", default="127.0.0.1:8000")
    p.add_argument("--device", type=int, default=0); p.add_argument("--max-context", type=int, default=32768)
    p.add_argument("--max-sequences", type=int, default=16); p.add_argument("--max-output", type=int, default=4096)
    p.add_argument("--pool-tokens", type=int, default=0); p.add_argument("--prefill-batch-tokens", type=int, default=4096)
    p.add_argument("--decode-share", type=float, default=0.2); p.add_argument("--prefix-cache-entries", type=int, default=20)
    p.add_argument("--prefix-cache-min-tokens", type=int, default=64); p.add_argument("--draft", default="ngram", choices=["off", "ngram", "mtp"])
    p.add_argument("--host-cache-gib", type=float, default=0.0, help="pinned host memory behind the prefix cache (0 = off)")
    p.add_argument("--host-cache-headroom-gib", type=float, default=0.0, help="part of --host-cache-gib left unused")
    p.add_argument("--host-cache-min-tokens", type=int, default=512, help="shorter prefixes are not written to the host tier")
    p.add_argument("--usage", default="off", choices=["on", "off"]); p.add_argument("--enable-bench", action="store_true")
    p.add_argument("--usage-dir", default=os.path.expanduser("~/.cache/cuteafd-b200/usage"))
    p.add_argument("--http-queue", type=int, default=64, help="requests that may wait for a lane; more are answered 429")
    p.add_argument("--queue-wait-s", type=float, default=0.0, help="admission wait budget in seconds (0 = wait as long as it takes)")
    p.add_argument("--gateway", default="on", choices=["on", "off"]); p.add_argument("--official-model-names", default="")
    p.add_argument("--official-model-names-file", default=""); p.add_argument("--gateway-allow-origin", default="")
    p.add_argument("--chat-template", default="", help="chat template family (chatml / qwen3-coder / deepseek / glm / plain); default: by model name")
    _gateway_args(p)
    p.add_argument("--draft-limit", type=int, default=3); p.add_argument("--api-key-file"); p.add_argument("--model-id")
    p.add_argument("--layers", type=int, default=0, help="debug: run only the first N layers of a named shape")
    p.add_argument("--n-micro", type=int, default=0, help="multi-GPU: micro-batches the attention ranks keep in flight (0 = the layout's default)")
    p.add_argument("--vision", default="auto", help="auto (tower of the snapshot, if it has one) | off | random[:DEPTH]")
    p.add_argument("--gpu-occupancy-percent", type=int, default=0,
                   help="size the KV pool by the capacity policy: share of the device this server may hold (0: --pool-tokens or 4096 pages as given)")
    p.add_argument("--draft-policy", default="simple", choices=["simple", "online"],
                   help="simple: fixed width with an acceptance cut-off; online: lengths of all requests chosen jointly from fitted round costs")
    p.add_argument("--audio", default="off", help="off | random[:DEPTH] (an audio encoder of the Whisper shape with random weights; `input_audio` parts accepted)")
    p.add_argument("--vision-max-patches", type=int, default=16384, help="patches of all images of one request")
    p.add_argument("--vision-max-images", type=int, default=8)
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("card")
    p.add_argument("--model", "--snapshot", dest="model", default="tiny"); p.add_argument("--device", type=int, default=0)
    p.add_argument("--max-context", type=int, default=16384); p.add_argument("--max-sequences", type=int, default=16)
    p.add_argument("--pool-tokens", type=int, default=0); p.add_argument("--prefill-batch-tokens", type=int, default=4096)
    p.add_argument("--decode-share", type=float, default=0.2); p.add_argument("--prefix-cache-entries", type=int, default=20)
    p.add_argument("--prefix-cache-min-tokens", type=int, default=64); p.add_argument("--draft", default="ngram", choices=["off", "ngram"])
    p.add_argument("--draft-limit", type=int, default=3); p.add_argument("--layers", type=int, default=0)
    p.add_argument("--c1-tokens", type=int, default=320); p.add_argument("--prefill-tokens", type=int, default=8192)
    p.add_argument("--golden", default=None, help="golden-window file: adds the logit-fidelity gate to the card's quality section")
    p.set_defaults(fn=cmd_card)
    p = sub.add_parser("gateway"); p.add_argument("--listen", default="127.0.0.1:8020"); p.add_argument("--model-id", default="cuteafd-b200")
    p.add_argument("--official-model-names", default=""); p.add_argument("--official-model-names-file", default="")
    p.add_argument("--gateway-allow-origin", default=""); p.add_argument("--chat-template", default="")
    p.add_argument("--replay", default="", help="replay a recorded JSONL session instead of serving; exit code 1 on differences")
    p.add_argument("--replay-url", default="", help="replay against this server instead of the in-process stand-in")
    _gateway_args(p); p.set_defaults(fn=cmd_gateway)
    p = sub.add_parser("quantize"); p.add_argument("src"); p.add_argument("dst")
    p.add_argument("--dense", default="nvfp4", choices=["bf16", "fp8_block128", "nvfp4", "mxfp4"])
    p.add_argument("--experts", default="mxfp4", choices=["bf16", "fp8_block128", "nvfp4", "mxfp4"])
    p.add_argument("--restart", action="store_true", help="discard a run store that belongs to another run"); p.set_defaults(fn=cmd_quantize)
    p = sub.add_parser("usage"); p.add_argument("action", choices=["clear", "clear-log", "export-csv", "demo"])
    p.add_argument("--dir", default=os.path.expanduser("~/.cache/cuteafd-b200/usage")); p.add_argument("--range", default="7d", choices=["1h", "6h", "24h", "7d"])
    p.add_argument("--out", default=""); p.add_argument("--listen", default="127.0.0.1:8010"); p.set_defaults(fn=cmd_usage)
    p = sub.add_parser("golden"); p.add_argument("--experts", default="bf16"); p.add_argument("--seed", type=int, default=0)
    p.add_argument("--write", default=None, help="seal golden windows of --model (tiny or a snapshot directory) into this file, from the fp32 oracle")
    p.add_argument("--check", default=None, help="check the GPU engine of --model against this golden file")
    p.add_argument("--model", "--snapshot", dest="model", default="tiny"); p.add_argument("--windows", type=int, default=8)
    p.add_argument("--window-tokens", type=int, default=64); p.set_defaults(fn=cmd_golden)
    p = sub.add_parser("expertd"); p.add_argument("--listen", default="127.0.0.1:7000"); p.add_argument("--rank", type=int, default=0); p.set_defaults(fn=cmd_expertd)
    p = sub.add_parser("bench"); p.add_argument("rest", nargs=argparse.REMAINDER); p.set_defaults(fn=cmd_bench)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
