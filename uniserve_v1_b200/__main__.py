"""Command line: ``python -m uniserve_v1_b200 serve PACKAGE [--ready-fd N] [--log-level L]``.

Like the reference's ``uniserve serve PACKAGE`` the command takes no deployment
option: everything is the package's ``config.toml`` (src/cli.rs:59-90, reference
project path).  ``build`` compiles the native libraries, ``layout`` prints the
resolved device layout of a package.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time


def serve(args) -> int:
    import torch
    import uvicorn

    from .checkpoint.safetensors_io import CheckpointLoader, resolve_family, resolve_hub
    from .config.policy import Package
    from .server.app import create_app

    pkg = Package.load(args.package)
    logging.basicConfig(level=getattr(logging, (args.log_level or pkg.logging_config.level).upper()))
    from .parallel.context import ParallelContext
    from .server import multirank as MR

    # One process per GPU: the serve command starts ranks 1..N-1 of the package's layout
    # itself (or joins a job started by a launcher that set RANK / WORLD_SIZE).
    par = MR.package_parallelism(pkg)
    want, axes = par["world"], par["axes"]
    union = MR.package_union(pkg)
    if union:
        want, axes = MR.package_world(pkg), {}
    cpu_ranks = os.environ.get("UNISERVE_CPU_RANKS", "0") == "1"     # gloo ranks, for tests
    children = []
    if want > 1 and "RANK" not in os.environ:
        have = torch.cuda.device_count() if torch.cuda.is_available() else 0
        if have >= want or cpu_ranks:
            import socket
            sock = socket.socket()
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
            sock.close()
            children = MR.spawn_followers(want, sys.argv[1:], port)
        else:
            logging.warning("layout wants %d ranks, %d GPUs present: serving on one rank", want,
                            have)
    rank, world, device, control = MR.init_rank()
    if cpu_ranks:
        device = torch.device("cpu")
    bus = MR.CommandBus(control, rank) if world > 1 else None
    dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[pkg.dtype]
    if device.type == "cpu":
        dtype = torch.float32
    directory = pkg.model_dir or None
    if directory is None and pkg.model and not pkg.model.startswith("random:"):
        directory = str(resolve_hub(pkg.model))
    family = "qwen3_moe"
    if directory:
        family = resolve_family(directory)
    elif pkg.model and "h3" in pkg.model.lower():
        family = "minimax_h3"
    elif pkg.model and "qwen4_exp" in pkg.model.lower():
        family = "qwen4_exp"
    name = pkg.served_model_name or (pkg.model or "model").split("/")[-1]
    shutdown = None
    if family == "minimax_h3":
        from .models.h3_vae import AudioVaeConfig, AudioVaeDecoder, VideoVaeConfig, VideoVaeDecoder
        from .models.minimax_h3 import H3Config, H3Transformer
        from .server.video_service import VideoService
        tiny = pkg.model and pkg.model.endswith(":tiny")
        cfg = H3Config.tiny() if tiny else H3Config()
        hybrid = axes.get("gather", 1) > 1 and axes.get("ulysses", 1) > 1
        seq = "sequence" if hybrid else ("gather" if "gather" in axes else "ulysses")
        if hybrid:
            ctx = ParallelContext.from_world(ulysses=axes["ulysses"], gather=axes["gather"])
        else:
            ctx = ParallelContext.from_world(**{seq: world}) if world > 1 else None
        tr = H3Transformer(cfg, device, dtype, ctx).init_random(0)
        if world > 1 and device.type == "cuda" and seq == "ulysses":
            from .parallel.ulysses import FusedUlysses
            from .server.video_rules import frames_for_seconds
            lf, lh, lw = cfg.latent_shape(frames_for_seconds(15), 1536, 768)
            # generated rows of the longest clip, then the prompt and the condition rows (two
            # keyframes and a dozen reference images at full raster fit; larger sets are refused)
            rows_max = (lf * (lh // 2) * (lw // 2) + cfg.audio_rows(frames_for_seconds(15)) +
                        16384 + 64 * world) // (64 * world) * (64 * world)
            tr.ulysses = FusedUlysses(ctx, device, rows_max, tr.heads_local, cfg.head_dim)
        vv = VideoVaeDecoder(VideoVaeConfig.tiny() if tiny else VideoVaeConfig(), device, dtype).init_random(1)
        if tiny:
            vv.cfg.latent_channels = cfg.latent_channels
            vv = VideoVaeDecoder(vv.cfg, device, dtype).init_random(1)
        av = AudioVaeDecoder(AudioVaeConfig.tiny() if tiny else AudioVaeConfig(), device).init_random(2)
        # the VAE's causal-convolution encoder turns first / last frame images into condition rows
        from .models.h3_vae_encoder import VideoEncoderConfig, VideoVaeEncoder
        ec = VideoEncoderConfig.tiny(cfg.latent_channels, cfg.vae_spatial) if tiny \
            else VideoEncoderConfig(latent_channels=cfg.latent_channels, tile=768, tile_overlap=128)
        from .models.h3_audio_encoder import AudioEncoderConfig, AudioVaeEncoder
        ac = AudioEncoderConfig.tiny(cfg.audio_channels) if tiny \
            else AudioEncoderConfig(latent_channels=cfg.audio_channels)
        service = VideoService(tr, vv, av, max_seconds=15,
                               retention_s=float(pkg.media_config.job_retention),
                               store_bytes=int(pkg.media_config.job_store_bytes),
                               video_encoder=VideoVaeEncoder(ec, device).init_random(3),
                               audio_encoder=AudioVaeEncoder(ac, device).init_random(4))
        if rank > 0:
            return 0 if MR.video_follower_loop(service, bus) >= 0 else 1
        if bus is not None:
            shutdown = MR.ReplicatedVideoService(service, bus).shutdown
        app = create_app(package=pkg, served_model_name=name, video_service=service)
    elif family == "qwen4_exp":
        # the hyper-connected decoder exists as FP32 formulas on the host only: a checkpoint's
        # or a random model of every part behind the usual routes, drafting with the MTP module
        # (the checkpoint's ``mtp.*``) when the package asks for draft tokens
        from .engine.dense_state import DenseStateEngine
        from .models.qwen4_exp import Qwen4ExpModel
        from .server.tokenizer import load_tokenizer
        assert world == 1, "this family is served on one rank"
        ld = None
        if directory:
            from .checkpoint.safetensors_io import CheckpointLoader
            ld = CheckpointLoader(directory)
            model = Qwen4ExpModel.from_checkpoint(ld)
        else:
            model = Qwen4ExpModel.tiny()

        def make_engine():
            return DenseStateEngine(model, max_num_seqs=min(pkg.max_running_requests,
                                                            pkg.scheduler_config.max_batch),
                                    max_model_len=pkg.max_model_len or 2048)
        tok = load_tokenizer(directory, model.cfg.vocab_size, model.cfg.eos_token_id)
        drafter = None
        if int(pkg.speculative_config.num_draft_tokens) > 0 and \
                (ld is None or ld.has("mtp.fc_hidden.weight")):
            from .models.qwen4_exp import Qwen4Mtp, Qwen4MtpDrafter
            mtp = Qwen4Mtp(model)
            mtp = mtp.load_state(ld) if ld is not None else mtp.init_random(1)
            drafter = Qwen4MtpDrafter(mtp, k=int(pkg.speculative_config.num_draft_tokens))
        app = create_app(package=pkg, engine=make_engine(), tokenizer=tok,
                         served_model_name=name, engine_factory=make_engine, drafter=drafter)
    elif family in ("qwen3_5_moe", "qwen3_vl"):
        # hybrid decoder (gated delta net + gated attention) or the dense Qwen3-VL language
        # model (three-axis positions, deep-stack inputs): dense per-sequence state
        from .checkpoint.quantized import open_checkpoint
        from .engine.dense_state import DenseStateEngine
        from .server.tokenizer import load_tokenizer
        assert world == 1, "this family is served on one GPU"
        ld = open_checkpoint(directory, dtype)
        if family == "qwen3_vl":
            from .models.qwen3_vl import Qwen3VLDenseModel, Qwen3VLTextConfig
            cfg = Qwen3VLTextConfig.from_hf(ld.config)
            model = Qwen3VLDenseModel(cfg, device, dtype).load_state(ld)
        else:
            from .models.qwen3_5 import Qwen35Config, Qwen35MoeModel
            cfg = Qwen35Config.from_hf(ld.config)
            model = Qwen35MoeModel(cfg, device, dtype).load_state(ld)

        tower = None
        if any(n.startswith("model.visual.") for n in ld.names()):      # image inputs
            from .models.qwen3_vl_vision import Qwen3VLVisionTower, VisionConfig
            tower = Qwen3VLVisionTower(VisionConfig.from_hf(ld.config), device,
                                       dtype).load_state(ld)

        def make_engine():
            return DenseStateEngine(model, max_num_seqs=min(pkg.max_running_requests,
                                                            pkg.scheduler_config.max_batch),
                                    max_model_len=pkg.max_model_len or 8192, tower=tower)
        tok = load_tokenizer(directory, cfg.vocab_size, cfg.eos_token_id)
        drafter = None
        k_draft = int(pkg.speculative_config.num_draft_tokens)
        if k_draft > 0 and family == "qwen3_5_moe" and ld.has("mtp.fc.weight"):
            from .models.qwen3_5 import HybridMtp, HybridMtpDrafter    # the checkpoint's drafter
            drafter = HybridMtpDrafter(HybridMtp(model).load_state(ld), k=k_draft)
        app = create_app(package=pkg, engine=make_engine(), tokenizer=tok,
                         served_model_name=name, engine_factory=make_engine, drafter=drafter)
    elif union and world > 1:
        # expert union: every attention member owns a scheduler and its requests, every MoE
        # layer is a lock-step exchange, steps are agreed over the control group
        from .engine.engine import LLMEngine
        from .engine.union import UnionFront, UnionMember, member_loop
        from .models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        from .server.tokenizer import load_tokenizer
        n_src = union["sources"]
        sources = tuple(range(n_src))
        experts = sources if union["shared"] else tuple(range(n_src, world))
        # `moe_config.exchange = "weights"`: distributed weight data parallelism - the members
        # keep their tokens and read the expert shards they miss from their peers
        dwdp = union["shared"] and (pkg.moe_config.exchange or "") == "weights"
        if dwdp:
            ctx = ParallelContext.from_world(expert=world)
        else:
            ctx = ParallelContext(world_rank=rank, world_size=world)
            ctx.source_ranks, ctx.expert_ranks = sources, experts
        if directory:
            from .checkpoint.quantized import open_checkpoint
            ld = open_checkpoint(directory, dtype)
            cfg = Qwen3MoeConfig.from_hf(ld.config)
            model = Qwen3MoeModel(cfg, device, dtype, ctx).load_state(ld)
        else:
            cfg = Qwen3MoeConfig.tiny() if (pkg.model or "").endswith(":tiny") \
                else Qwen3MoeConfig.qwen3_30b_a3b()
            model = Qwen3MoeModel(cfg, device, dtype, ctx).init_random(0)
        limit = min(int(pkg.max_num_batched_tokens or 8192), 8192)
        if dwdp:
            import torch.distributed as dist
            from .parallel.dwdp import attach_weight_peers
            attach_weight_peers(model, dist.group.WORLD if device.type == "cuda" else control,
                                rank, world)
        elif device.type == "cuda":
            import torch.distributed as dist
            from .parallel.expert_exchange import ExpertExchange
            model.exchange = ExpertExchange(dist.group.WORLD, rank, world, device, limit,
                                            cfg.num_experts_per_tok, cfg.hidden_size,
                                            cfg.num_experts, cfg.moe_intermediate_size,
                                            sources, experts)
        else:
            from .parallel.expert_exchange import HostExpertExchange
            model.exchange = HostExpertExchange(control, rank, world, limit,
                                                cfg.num_experts_per_tok, cfg.hidden_size,
                                                cfg.num_experts, sources, experts)
        mb = int(pkg.moe_config.microbatches or 1)
        if mb >= 2 and not dwdp and not union["shared"]:
            # (members that hold experts themselves gain nothing: the same GPU would read the
            # expert weights twice per layer - measured 22.8 against 12.3 ms per step)
            # two more exchanges of half the window each: decode steps run as two interleaved
            # half-batches (attention of one under the experts of the other)
            half = max(1, limit // 2)
            if device.type == "cuda":
                import torch.distributed as dist
                from .parallel.expert_exchange import ExpertExchange
                model.micro_exchanges = [
                    ExpertExchange(dist.group.WORLD, rank, world, device, half,
                                   cfg.num_experts_per_tok, cfg.hidden_size, cfg.num_experts,
                                   cfg.moe_intermediate_size, sources, experts) for _ in (0, 1)]
            else:
                from .parallel.expert_exchange import HostExpertExchange
                model.micro_exchanges = [
                    HostExpertExchange(control, rank, world, half, cfg.num_experts_per_tok,
                                       cfg.hidden_size, cfg.num_experts, sources, experts)
                    for _ in (0, 1)]
        eng = None
        if rank in sources:
            eng = LLMEngine(model,
                            page_size=min(pkg.kv_cache_config.block_size, 16)
                            if device.type == "cuda" else pkg.kv_cache_config.block_size,
                            max_num_seqs=min(pkg.max_running_requests, pkg.scheduler_config.max_batch),
                            max_model_len=pkg.max_model_len or min(cfg.max_position_embeddings, 8192),
                            max_num_batched_tokens=limit,
                            mem_fraction_static=pkg.mem_fraction_static,
                            enable_prefix_cache=pkg.kv_cache_config.prefix_caching,
                            watchdog_timeout=float(pkg.profiling_config.watchdog_timeout),
                            **({"num_pages": 512, "use_graphs": False} if device.type == "cpu"
                               else ({"use_graphs": False} if dwdp else {})))
        member = UnionMember(control, rank, world, sources, experts, engine=eng, model=model,
                             capacity_limit=limit,
                             exchange_free=dwdp and device.type == "cuda", microbatches=mb)
        if rank > 0:
            member_loop(member, 0)
            return 0
        tok = load_tokenizer(directory, cfg.vocab_size, cfg.eos_token_id)
        front = UnionFront(member, 0)
        shutdown = front.shutdown
        app = create_app(package=pkg, engine=front, tokenizer=tok, served_model_name=name)
    else:
        from .engine.engine import LLMEngine
        from .models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
        from .server.tokenizer import load_tokenizer
        ctx = None
        if world > 1:
            pp = axes.get("layer", 1) if world % axes.get("layer", 1) == 0 else 1
            ctx = ParallelContext.from_world(tensor=world // pp, layer=pp,
                                             expert_over_tensor=world // pp > 1)
        cfg, model, ld = _qwen3_model(pkg, directory, device, dtype, ctx,
                                      getattr(args, "weights_socket", None))
        if pkg.profiling_config.expert_load and hasattr(model, "enable_expert_load") and \
                (device.type == "cpu" or "expert_order" in pkg.programs
                 or os.environ.get("US_EXPERT_LOAD") == "1"):
            # tokens per expert and routed layer (uniserve_expert_tokens_total): on a GPU the
            # counting costs launches, so it runs while the package's program reads it
            model.enable_expert_load()
        if ctx is not None and ctx.tp_size > 1 and device.type == "cuda":
            from .parallel.symm import attach_fused
            attach_fused(ctx, device, hidden=cfg.hidden_size)
            from .parallel.tp_fused import attach_fused_tp      # prefill chunks: fused RS / AG
            attach_fused_tp(model, int(pkg.max_num_batched_tokens or 8192))

        def make_engine(pkg=pkg):
            from .engine.quota import quota_of
            policy = None
            if "scheduling" in pkg.programs:        # the package's own scheduling program
                from .engine.program import ProgramHost, ProgramPolicy
                policy = ProgramPolicy(ProgramHost.load(pkg, "scheduling"))
            eng = LLMEngine(model, policy=policy,
                            page_size=min(pkg.kv_cache_config.block_size, 16)
                            if device.type == "cuda" else pkg.kv_cache_config.block_size,
                            max_num_seqs=min(pkg.max_running_requests, pkg.scheduler_config.max_batch),
                            max_model_len=pkg.max_model_len or min(cfg.max_position_embeddings, 8192),
                            max_num_batched_tokens=pkg.max_num_batched_tokens,
                            mem_fraction_static=pkg.mem_fraction_static,
                            enable_prefix_cache=pkg.kv_cache_config.prefix_caching,
                            host_kv_ratio=(pkg.kv_cache_config.host_ratio
                                           if pkg.kv_cache_config.host_tier else 0.0),
                            host_kv_gib=pkg.kv_cache_config.host_gib,
                            host_reserve_gib=float(pkg.storage_config.host_reserve_gib),
                            watchdog_timeout=float(pkg.profiling_config.watchdog_timeout),
                            kv_dtype=pkg.kv_cache_config.dtype,
                            # an engine built beside one that serves (the target of an epoch
                            # update) must fit what is left of the device's quota
                            quota_strict=quota_of(device).usage() > 0,
                            **({"num_pages": 512, "use_graphs": False} if device.type == "cpu" else {}))
            return MR.ReplicatedEngine(eng, bus) if bus is not None and rank == 0 else eng

        if rank > 0:
            MR.follower_loop(make_engine(), bus)
            return 0
        tok = load_tokenizer(directory, cfg.vocab_size, cfg.eos_token_id)
        engine = make_engine()
        if bus is not None:
            shutdown = engine.shutdown
        if getattr(args, "prefix_cache", None) and bus is None:
            from .engine.prefix_store import load_prefix_cache
            got = load_prefix_cache(engine, args.prefix_cache)
            print(f"prefix cache: {got}", file=sys.stderr)
        sess = pkg.profiling_config.session
        if sess.collectors and bus is None:
            # a package that names session collectors starts profiling with the deployment
            from .engine.profiling import start_session
            st = start_session(engine, list(sess.collectors), sess.output,
                               seconds=float(sess.duration) if sess.duration else None, rank=rank)
            print(f"profile session: {st['path']} ({', '.join(st['collectors'])})", file=sys.stderr)
        # a replicated engine cannot be rebuilt on one rank alone: no in-place restart
        drafter = None
        k_draft = int(pkg.speculative_config.num_draft_tokens)
        if k_draft > 0 and bus is None and directory and ld.has("mtp.fc.weight"):
            from .models.qwen3_mtp import MtpDrafter, MtpHead     # the checkpoint's own drafter
            drafter = MtpDrafter(MtpHead(model).load_state(ld), k=k_draft)
        # prefill / decode role of this replica: `--role`, or `replicas.<id>.role` of the
        # package for `--replica-id`; the internal routes need UNISERVE_INTERNAL_KEY
        role = args.role or (pkg.replicas[args.replica_id].role if args.replica_id else "mixed")
        app = create_app(package=pkg, engine=engine, tokenizer=tok, served_model_name=name,
                         engine_factory=make_engine if bus is None else None, drafter=drafter,
                         role=role, internal_key=os.environ.get("UNISERVE_INTERNAL_KEY"),
                         # epoch updates build the target engine (a second scheduler and KV
                         # cache over the same weights) beside the serving one
                         engine_builder=make_engine if bus is None else None,
                         state_dir=getattr(args, "state_dir", None))
    # The listening socket is this process's own object (not uvicorn's), so that a successor
    # started by `POST /admin/restart` can inherit it: no connection is refused while the
    # deployment changes hands.
    import socket as _socket
    listener = None
    if getattr(args, "listen_fd", None) is not None:
        listener = _socket.socket(fileno=args.listen_fd)          # handed over by a predecessor
    elif not pkg.admin_config.uds:
        listener = _socket.socket(_socket.AF_INET, _socket.SOCK_STREAM)
        listener.setsockopt(_socket.SOL_SOCKET, _socket.SO_REUSEADDR, 1)
        listener.bind((pkg.admin_config.host, pkg.admin_config.port or 8000))
        listener.listen(2048)
    if listener is not None:
        listener.set_inheritable(True)
    config = uvicorn.Config(app, host=pkg.admin_config.host, port=pkg.admin_config.port or 8000,
                            uds=pkg.admin_config.uds if listener is None else None,
                            fd=listener.fileno() if listener is not None else None,
                            log_level=(args.log_level_http or pkg.logging_config.http_level
                                       or "warning"),
                            h11_max_incomplete_event_size=int(pkg.server_config.max_request_head))
    server = uvicorn.Server(config)
    standby = None
    if world == 1 and listener is not None:
        from .server.restart import HotRestart, Standby, park
        app.state.generation = int(getattr(args, "generation", 0) or 0)
        snapshot = None
        svc = getattr(app.state.s, "service", None)
        if svc is not None and hasattr(getattr(app.state.s, "engine", None), "blocks"):
            from .engine.prefix_store import default_path, save_prefix_cache

            def snapshot():
                # the successor starts with this process's cached prefixes
                path = default_path(getattr(args, "state_dir", None), app.state.generation)
                return svc.call(lambda e: save_prefix_cache(e, path))["path"]
        app.state.restart = HotRestart(server, listener, sys.argv[1:], snapshot=snapshot)
        if getattr(args, "standby_fd", None) is not None:
            # this process is a standby: park until the serving process ends
            eng = getattr(app.state.s, "engine", None)
            from .server.restart import PrefixSnapshots
            if not park(args.standby_fd, args.ready_fd, eng,
                        pkg.profiling_config.standby_storage,
                        PrefixSnapshots.path_for(listener, getattr(args, "state_dir", None))):
                return 0
            args.ready_fd = None
        if pkg.profiling_config.standby:
            standby = Standby(listener, sys.argv[1:], app.state.generation)
            standby.start()
            app.state.standby = standby
            period = float(pkg.profiling_config.standby_snapshot)
            if period > 0 and svc is not None and hasattr(getattr(app.state.s, "engine", None),
                                                          "blocks"):
                from .server.restart import PrefixSnapshots
                snaps = PrefixSnapshots(svc, PrefixSnapshots.path_for(
                    listener, getattr(args, "state_dir", None)), period)
                snaps.start()
                app.state.prefix_snapshots = snaps
    supervision = None
    if children and listener is not None:
        # the leader watches the ranks it started; a rank that ends takes the deployment
        # through a relaunch on the same socket
        from .server.restart import Supervision
        app.state.generation = int(getattr(args, "generation", 0) or 0)

        def rank_failed(why):
            eng = getattr(app.state.s, "engine", None)
            if eng is not None:
                try:
                    eng.failed = f"fatal_worker_failure: {why}"
                except Exception:
                    pass
        supervision = Supervision(children, listener, sys.argv[1:], app.state.generation,
                                  on_failure=rank_failed,
                                  relaunch=os.environ.get("UNISERVE_RELAUNCH", "1") == "1",
                                  restart_s=float(pkg.storage_config.child_restart_s),
                                  restart_max_s=float(pkg.storage_config.child_restart_max_s))
        supervision.start()
        app.state.supervision = supervision
    if args.ready_fd is not None:
        os.write(args.ready_fd, json.dumps({"state": "listening", "host": pkg.admin_config.host,
                                            "port": pkg.admin_config.port,
                                            "pid": os.getpid()}).encode() + b"\n")
    try:
        server.run()
    finally:
        if supervision is not None:
            supervision.stop()
        if standby is not None and not getattr(app.state.restart, "state", "") == "failed":
            standby.stop()
        if shutdown is not None:
            shutdown()
        for c in children:
            try:
                c.wait(timeout=30)
            except Exception:
                c.terminate()
    return 0


def _qwen3_model(pkg, directory, device, dtype, ctx, weights_socket=None):
    """The package's Qwen3 model: mapped from a weights keeper when one answers on
    ``weights_socket`` with this model's identity, else read from the checkpoint (or drawn
    at random for ``random:`` models).  Returns (config, model, checkpoint loader or None)."""
    from .models.qwen3_moe import Qwen3MoeConfig, Qwen3MoeModel
    ld = None
    if directory:
        from .checkpoint.quantized import open_checkpoint
        ld = open_checkpoint(directory, dtype)       # NVFP4 / FP8 exports expand on read
        cfg = Qwen3MoeConfig.from_hf(ld.config)
    else:
        cfg = Qwen3MoeConfig.tiny() if (pkg.model or "").endswith(":tiny") \
            else Qwen3MoeConfig.qwen3_30b_a3b()
    model = Qwen3MoeModel(cfg, device, dtype, ctx)
    if weights_socket:
        from .server.weights_keeper import attach
        if attach(model, weights_socket):
            logging.info("weights mapped from the keeper at %s (%s)", weights_socket,
                         model.weights_from)
            return cfg, model, ld
        logging.warning("no weights keeper with this model at %s: loading", weights_socket)
    model = model.load_state(ld) if directory else model.init_random(0)
    return cfg, model, ld


def keep(args) -> int:
    """``keep PACKAGE --socket PATH``: hold the package's weights for serving processes."""
    import torch
    from .checkpoint.safetensors_io import resolve_hub
    from .config.policy import Package
    from .server.weights_keeper import WeightsKeeper
    pkg = Package.load(args.package)
    logging.basicConfig(level=logging.INFO)
    cpu = os.environ.get("UNISERVE_CPU_RANKS", "0") == "1" or not torch.cuda.is_available()
    device = torch.device("cpu") if cpu else torch.device("cuda", 0)
    dtype = torch.float32 if cpu else {"bfloat16": torch.bfloat16, "float16": torch.float16,
                                       "float32": torch.float32}[pkg.dtype]
    directory = pkg.model_dir or None
    if directory is None and pkg.model and not pkg.model.startswith("random:"):
        directory = str(resolve_hub(pkg.model))
    _cfg, model, _ld = _qwen3_model(pkg, directory, device, dtype, None)
    keeper = WeightsKeeper(model, args.socket)

    def ready():
        if args.ready_fd is not None:
            os.write(args.ready_fd, json.dumps({"state": "keeping", "pid": os.getpid(),
                                                "tensors": len(keeper.records)}).encode() + b"\n")
    keeper.serve_forever(ready)
    return 0


def admin(args) -> int:
    """Admin client over plain HTTP (crates/manager/src/main.rs:1-25, reference project
    path): prints the server's JSON answer; exit status 1 on an HTTP error.  ``status``,
    ``watch`` and ``apply`` take several ``--url`` and treat them as one deployment: the state
    of every node in one table, a line per change, and a policy put on every node with the
    nodes already changed put back when one refuses."""
    import urllib.error
    import urllib.request
    head = {"Authorization": f"Bearer {args.api_key}"} if args.api_key else {}
    urls = args.url or ["http://127.0.0.1:8000"]

    def call(url, path, data=None, method=None, ctype=None, timeout=60):
        h = dict(head, **({"Content-Type": ctype} if ctype else {}))
        req = urllib.request.Request(url + path, data=data, method=method, headers=h)
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.read().decode()

    def node_state(url) -> dict:
        row = {"url": url}
        try:
            h = json.loads(call(url, "/health", timeout=10))
            row.update(status=h.get("status"), pid=h.get("pid"), generation=h.get("generation"),
                       asleep=h.get("asleep"), uptime_s=round(h.get("uptime_seconds", 0.0), 1))
        except urllib.error.HTTPError as e:
            row.update(status=f"http {e.code}")
            return row
        except Exception as e:
            row.update(status="unreachable", error=type(e).__name__)
            return row
        try:
            pol = json.loads(call(url, "/admin/policy", timeout=10))
            row.update(revision=pol.get("revision"), model=pol.get("config", {}).get("served_model_name"),
                       paused=pol.get("config", {}).get("paused"))
        except Exception:
            pass
        return row

    if args.verb == "status":
        rows = [node_state(u) for u in urls]
        print(json.dumps(rows, indent=1))
        return 0 if all(r.get("status") == "ok" for r in rows) else 1
    if args.verb == "watch":
        # one line per node whose state changed; --count polls (0 = until interrupted)
        last, n = {}, 0
        try:
            while True:
                for u in urls:
                    row = node_state(u)
                    key = {k: v for k, v in row.items() if k != "uptime_s"}
                    if last.get(u) != key:
                        last[u] = key
                        print(json.dumps(dict(row, at=round(time.time(), 1))), flush=True)
                n += 1
                if args.count and n >= args.count:
                    return 0
                time.sleep(args.interval)
        except KeyboardInterrupt:
            return 0
    if args.verb == "apply":
        body = open(args.arg, "rb").read()
        before, done = {}, []
        for u in urls:              # what to put back if a later node refuses
            try:
                before[u] = json.loads(call(u, "/admin/policy", timeout=10)).get("toml")
            except Exception:
                before[u] = None
        for u in urls:
            try:
                out = call(u, "/admin/policy", data=body, method="PUT", ctype="application/toml")
                done.append(u)
                print(json.dumps({"url": u, "applied": json.loads(out).get("revision")}))
            except urllib.error.HTTPError as e:
                print(json.dumps({"url": u, "refused": e.read().decode()[:400]}), file=sys.stderr)
                for d in done:      # the nodes already changed return to what they served
                    if before.get(d):
                        try:
                            call(d, "/admin/policy", data=before[d].encode(), method="PUT",
                                 ctype="application/toml")
                            print(json.dumps({"url": d, "restored": True}))
                        except Exception as e2:
                            print(json.dumps({"url": d, "restored": False, "error": str(e2)}),
                                  file=sys.stderr)
                return 1
        return 0
    url = urls[0]
    try:
        if args.verb == "get-policy":
            print(call(url, "/admin/policy"))
        elif args.verb == "health":
            print(call(url, "/health"))
        elif args.verb == "put-policy":
            print(call(url, "/admin/policy", data=open(args.arg, "rb").read(), method="PUT",
                       ctype="application/toml"))
        else:
            print(call(url, "/admin/query", data=(args.arg or "").encode(), method="POST",
                       ctype="text/plain"))
        return 0
    except urllib.error.HTTPError as e:
        print(e.read().decode(), file=sys.stderr)
        return 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="uniserve_v1_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="serve a policy package")
    s.add_argument("package")
    s.add_argument("--ready-fd", type=int, default=None)
    s.add_argument("--weights-socket", default=None,
                   help="map the weights from a `keep` process on this unix socket when it answers")
    s.add_argument("--standby-fd", type=int, default=None,
                   help="park as a standby until this pipe closes (the serving process ended)")
    s.add_argument("--generation", type=int, default=0, help="launch generation (standbys count up)")
    s.add_argument("--listen-fd", type=int, default=None,
                   help="an already listening socket handed over by the process this one replaces")
    s.add_argument("--log-level", default=None)
    s.add_argument("--log-level-http", default=None)
    s.add_argument("--prefix-cache", default=None,
                   help="file of a predecessor's cached KV pages to read before serving "
                        "(written at a hot restart; removed once read)")
    s.add_argument("--state-dir", default=None,
                   help="directory where control programs keep their state across restarts")
    s.add_argument("--role", choices=["mixed", "prefill", "decode"], default=None,
                   help="disaggregation role of this replica (default: the package's "
                        "replicas.<id>.role for --replica-id, else mixed)")
    s.add_argument("--replica-id", default=None, help="key of this replica in [replicas]")
    k = sub.add_parser("keep", help="hold a package's weights for serving processes to map")
    k.add_argument("package")
    k.add_argument("--socket", required=True, help="unix socket the keeper answers on")
    k.add_argument("--ready-fd", type=int, default=None)
    b = sub.add_parser("build", help="compile the native libraries for sm_100a")
    b.add_argument("--force", action="store_true")
    l = sub.add_parser("layout", help="print the resolved device layout of a package")
    l.add_argument("package")
    ad = sub.add_parser("admin", help="admin client: policy get / put, SQL query")
    ad.add_argument("--url", action="append", default=None,
                    help="node address (repeat for status / watch / apply over several nodes)")
    ad.add_argument("--api-key", default=None)
    ad.add_argument("--interval", type=float, default=2.0, help="watch: seconds between polls")
    ad.add_argument("--count", type=int, default=0, help="watch: polls before it ends (0: none)")
    ad.add_argument("verb", choices=["get-policy", "put-policy", "query", "health", "status",
                                     "watch", "apply"])
    ad.add_argument("arg", nargs="?", help="config.toml to put / apply, or the SQL text")
    r = sub.add_parser("route", help="one address in front of data-parallel replicas")
    r.add_argument("--listen", default="127.0.0.1:8000")
    r.add_argument("--replica", action="append", default=[], help="base URL of a mixed replica")
    r.add_argument("--prefill", action="append", default=[], help="base URL of a prefill replica")
    r.add_argument("--decode", action="append", default=[], help="base URL of a decode replica")
    r.add_argument("--program", help="routing program: a file that defines route(request, replicas)")
    r.add_argument("--internal-key", default=os.environ.get("UNISERVE_INTERNAL_KEY"),
                   help="key presented to prefill / decode replicas on their internal routes")
    r.add_argument("--prefix-aware", action="store_true",
                   help="ask the replicas which of them holds a request's prompt prefix and "
                        "send it there (requests without prompt_cache_key)")
    r.add_argument("--transfer-deadline", type=float, default=60.0, metavar="SECONDS",
                   help="time each leg of a prefill -> decode hand-off may take (504 after it)")
    a = ap.parse_args(argv)
    if a.cmd == "serve":
        return serve(a)
    if a.cmd == "keep":
        return keep(a)
    if a.cmd == "admin":
        return admin(a)
    if a.cmd == "route":
        import uvicorn
        from .server.router import create_router_app
        host, _, port = a.listen.rpartition(":")
        if not a.replica and not (a.prefill and a.decode):
            ap.error("route needs --replica, or --prefill together with --decode")
        program = None
        if a.program:
            from .engine.program import ProgramHost
            program = ProgramHost(open(a.program).read(), "routing", call_fuel=1_000_000)
        uvicorn.run(create_router_app(a.replica, prefill_urls=a.prefill or None,
                                      decode_urls=a.decode or None, program=program,
                                      internal_key=a.internal_key,
                                      prefix_aware=a.prefix_aware,
                                      transfer_deadline_s=a.transfer_deadline),
                    host=host or "127.0.0.1", port=int(port), log_level="warning")
        return 0
    if a.cmd == "build":
        from . import build
        print(build.build(force=a.force)["kernels"])
        return 0
    from .config.policy import Package
    print(json.dumps(Package.load(a.package).layout(), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
