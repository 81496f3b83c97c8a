"""``python -m tensorsharp_b200.server --model x.gguf [--backend b200|cpu] [--port 5000] ...``

Parity: TensorSharp.Server/Program.cs, Hosting/StartupBanner.cs, StartupModelLoader.cs,
LoggingSetup.cs: build the options, set up the JSONL log, print the banner, load the hosted
model (when ``--model`` was given) and warm its kernels up, then serve.
"""
from __future__ import annotations

import os
import sys
import time

from ..runtime import media
from ..runtime.logging import Ev, setup_file_logging
from .app import ServerApp, serve
from .options import build_options, read_configured_backend_input, try_resolve_supported_backend

ENDPOINT_SUMMARY = (
    "GET  /                         - Health check",
    "GET  /metrics                   - Serving totals (Prometheus text format)",
    "GET  /api/tags                  - List hosted models (Ollama)",
    "POST /api/show                  - Show model details (Ollama)",
    "POST /api/generate              - Generate text (Ollama)",
    "POST /api/chat/ollama           - Chat completion (Ollama)",
    "POST /v1/chat/completions       - Chat completion (OpenAI)",
    "GET  /v1/models                 - List hosted models (OpenAI)",
    "POST /api/chat                  - Chat (Web UI SSE)",
    "POST /api/models/load           - Reload hosted model (Web UI)",
    "GET  /api/models                - Show hosted model state (Web UI)",
)

USAGE = ("No startup model configured. Launch with --model <path.gguf> --backend <type> [--mmproj <path>] "
         "[--max-tokens 20000] [--temperature F] [--top-k N] [--top-p F] [--min-p F] [--repeat-penalty F] "
         "[--presence-penalty F] [--frequency-penalty F] [--seed N] [--stop <text>] [--max-context N] [--kv-dtype bf16|fp8] [--max-sessions N] "
         "[--max-batch N] [--replicas N] to use the Web UI.")


def _fmt(v: float) -> str:
    return ("%.3f" % v).rstrip("0").rstrip(".") or "0"


def emit_banner(log, options, listen: str, out=sys.stdout) -> None:
    def info(ev, template, **kw):
        log.info(ev, template, **kw)
        print(template.format(**kw), file=out)
    if not options.supported_backends:
        log.warning(Ev.BackendUnavailable, "No supported backends detected on this machine.")
    else:
        info(Ev.BackendDetected, "Supported backends: {SupportedBackends}",
             SupportedBackends=", ".join(b["value"] for b in options.supported_backends))
    info(Ev.HostConfiguration, "Server configuration: hostedModel={HostedModel} hostedMmProj={HostedMmProj} "
         "defaultWebMaxTokens={DefaultWebMaxTokens} videoMaxFrames={VideoMaxFrames} listen={ListenAddress}",
         HostedModel=options.startup_model_path or "(none)", HostedMmProj=options.startup_mmproj_path or "(none)",
         DefaultWebMaxTokens=options.default_web_max_tokens, VideoMaxFrames=media.get_configured_max_video_frames(),
         ListenAddress=listen)
    s = options.default_sampling_config
    info(Ev.HostConfiguration, "Default sampling: temperature={Temperature} topK={TopK} topP={TopP} minP={MinP} "
         "repeatPenalty={RepeatPenalty} presencePenalty={PresencePenalty} frequencyPenalty={FrequencyPenalty} seed={Seed} "
         "stopSequences={StopSequences}", Temperature=_fmt(s.temperature), TopK=s.top_k, TopP=_fmt(s.top_p),
         MinP=_fmt(s.min_p), RepeatPenalty=_fmt(s.repetition_penalty), PresencePenalty=_fmt(s.presence_penalty),
         FrequencyPenalty=_fmt(s.frequency_penalty), Seed=s.seed,
         StopSequences="[" + ", ".join('"%s"' % x for x in s.stop_sequences) + "]" if s.stop_sequences else "(none)")
    info(Ev.HostStarting, "Starting TensorSharp.Server on {ListenAddress}", ListenAddress=listen)
    for ep in ENDPOINT_SUMMARY:
        info(Ev.HostConfiguration, "Endpoint: {Endpoint}", Endpoint=ep)


def load_startup_model(options, svc, configured_backend, log) -> None:
    if not options.startup_model_path:
        log.info(Ev.HostConfiguration, USAGE)
        print(USAGE)
        return
    backend, err = try_resolve_supported_backend(options, configured_backend)
    if err:
        raise RuntimeError(err)
    if not os.path.isfile(options.startup_model_path):
        raise FileNotFoundError(f"Configured model file not found: {options.startup_model_path}")
    if options.startup_mmproj_path and not os.path.isfile(options.startup_mmproj_path):
        raise FileNotFoundError(f"Configured mmproj file not found: {options.startup_mmproj_path}")
    svc.load_model(options.startup_model_path, options.startup_mmproj_path, backend)
    log.info(Ev.ModelLoadCompleted, "Startup model loaded: {Model} architecture={Architecture} backend={Backend} mmproj={MmProj}",
             Model=svc.loaded_model_name, Architecture=svc.architecture or "unknown", Backend=svc.loaded_backend,
             MmProj=svc.loaded_mmproj_name or "(none)")
    warm = getattr(svc.model, "warm_up_kernels", None)
    if warm is not None:
        t0 = time.perf_counter()
        warm()
        log.info(Ev.HostConfiguration, "Kernel warmup completed in {ElapsedMs:.1f} ms", ElapsedMs=(time.perf_counter() - t0) * 1e3)


def run_replicated(argv, options) -> int:
    """``--replicas N``: N server processes (one per GPU) and the routing front end on the public address."""
    from .replicas import Router, Supervisor, serve_front, spawn_replicas, stop_replicas
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print("error: --replicas starts its own processes; do not combine it with torch.distributed.run", file=sys.stderr)
        return 2
    backend = try_resolve_supported_backend(options, read_configured_backend_input(argv))[0] or "cpu"
    log_dir = options.log_directory if options.file_logging_enabled else None
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
    import signal

    def on_term(signum, frame):                  # end like Ctrl-C so that the replica processes are stopped too
        raise KeyboardInterrupt
    signal.signal(signal.SIGTERM, on_term)
    replicas = spawn_replicas(argv, options.replicas, use_gpus=backend != "cpu", log_dir=log_dir)
    router = Router(replicas)
    supervisor = Supervisor(router).start()          # a replica that dies is started again
    front = serve_front(router, options.host, options.port)
    print(f"{len(replicas)} replicas ready ({', '.join(str(r.port) for r in replicas)}); listening on "
          f"http://{options.host}:{front.server_address[1]}", flush=True)
    try:
        front.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        supervisor.stop()
        front.server_close()
        stop_replicas(replicas)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    base = os.environ.get("TENSORSHARP_BASE_DIR") or os.getcwd()
    try:
        options = build_options(argv, base)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if options.replicas > 1:
        return run_replicated(argv, options)
    # A model over several processes: started as ``python -m torch.distributed.run --nproc-per-node N -m tensorsharp_b200.server ...``
    # every process holds its part (``--parallel tp`` weight shards, ``pp`` layer ranges, ``cp`` whole copies that share long
    # prompts); rank 0 runs the HTTP front end and announces each model call, the others mirror it.
    comm = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from ..parallel.dist import init_from_env
        from ..parallel.replicated import follower_main, layout_create, leader_factory, shutdown_followers
        cpu_only = (try_resolve_supported_backend(options, read_configured_backend_input(argv))[0] or "") == "cpu"
        comm = init_from_env("gloo" if cpu_only else None)
        create = layout_create(options.parallel)
        from ..parallel.replicated import start_watchdog
        hb_timeout = float(os.environ.get("TSB_WATCHDOG_S", "30") or 0)
        if comm.rank != 0:
            def leader_gone(stale):              # rank 0 went quiet: nothing will ever tell this process to stop
                if 0 in stale:
                    print(f"rank {comm.rank}: the front end (rank 0) stopped answering; exiting", file=sys.stderr, flush=True)
                    os._exit(3)
            start_watchdog(comm, hb_timeout, on_failure=leader_gone)
            follower_main(comm, create=create)
            return 0
        watchdog = start_watchdog(comm, hb_timeout)
    provider = setup_file_logging(options.log_directory, prefix="tensorsharp-server", enabled=options.file_logging_enabled)
    svc = None
    if comm is not None:
        from .model_service import ModelService
        svc = ModelService(None, model_factory=leader_factory(comm, create, watchdog), max_context=options.max_context,
                           max_sessions=options.max_sessions)
    app = ServerApp(options, svc=svc, log_provider=provider)
    log = app.logger("TensorSharp.Server")
    listen = f"http://{options.host}:{options.port}"
    emit_banner(log, options, listen)
    load_startup_model(options, app.svc, read_configured_backend_input(argv), log)
    httpd = serve(app)
    log.info(Ev.HostStarted, "TensorSharp.Server listening on {ListenAddress}", ListenAddress=listen)
    from ..runtime.banner import print_banner
    print_banner(["B200-native GGUF inference server", f"model: {app.svc.loaded_model_name or '(none loaded)'}",
                  f"backend: {app.svc.loaded_backend or '(none)'}"])
    print(f"listening on {listen}")
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        log.info(Ev.HostStopping, "TensorSharp.Server stopping")
        httpd.server_close()
        app.svc.close()
        if comm is not None:
            shutdown_followers(comm)
        log.info(Ev.HostStopped, "TensorSharp.Server stopped")
        if provider is not None:
            provider.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
