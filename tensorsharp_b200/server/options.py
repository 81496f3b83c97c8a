"""Server configuration: command line + environment, backend catalogue, hosted-model guard.

Parity: TensorSharp.Server/Hosting/ServerOptionsBuilder.cs (flags ``--model --mmproj --backend
--max-tokens --temperature --top-k --top-p --min-p --repeat-penalty --presence-penalty
--frequency-penalty --seed --stop`` in ``--flag value`` or ``--flag=value`` form, flag names
case-insensitive; environment ``BACKEND MAX_TOKENS MAX_TEXT_FILE_CHARS TENSORSHARP_LOG_DIR
TENSORSHARP_LOG_FILE TENSORSHARP_TEMPERATURE TENSORSHARP_TOP_K ...``; a flag beats the
environment, which beats the built-in default), BackendCatalog.cs, Hosting/BackendSelector.cs,
Hosting/HostedModelGuard.cs.

Backends here are ``b200`` (the sm_100a kernels) and ``cpu`` (the fp32 oracle path); the
reference's names ``cuda`` / ``ggml_cuda`` are accepted as aliases of ``b200`` and
``ggml_cpu`` of ``cpu`` so existing launch scripts keep working.  This build adds
``--host --port --max-context --kv-dtype --max-sessions --max-batch --replicas --parallel`` (tensor parallelism comes from the
process count of the launch).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..runtime.sampling import SamplingConfig

DEFAULT_WEB_MAX_TOKENS = 20000
DEFAULT_MAX_TEXT_FILE_CHARS = 8000

BACKENDS: Tuple[Tuple[str, str, bool], ...] = (
    ("b200", "B200 (sm_100a CUDA)", False),
    ("cpu", "CPU (PyTorch fp32)", True),
)
_ALIASES = {"cuda": "b200", "ggml_cuda": "b200", "gpu": "b200", "b200": "b200", "ggml_cpu": "cpu", "cpu": "cpu"}


def canonicalize_backend(backend: Optional[str]) -> Optional[str]:
    if backend is None or not backend.strip():
        return None
    v = backend.strip().lower()
    return _ALIASES.get(v, v)


def _cuda_available() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def supported_backends(is_available: Optional[Callable[[str], bool]] = None) -> List[Dict[str, str]]:
    is_available = is_available or (lambda name: _cuda_available())
    return [{"value": v, "label": l} for v, l, always in BACKENDS if always or is_available(v)]


def resolve_default_backend(configured: Optional[str], supported: Sequence[Dict[str, str]]) -> Optional[str]:
    c = canonicalize_backend(configured)
    if c and any(b["value"].lower() == c for b in supported):
        return c
    return supported[0]["value"] if supported else (c or configured)


def backend_device(backend: Optional[str]) -> str:
    return "cuda" if canonicalize_backend(backend) == "b200" else "cpu"


@dataclass
class ServerHostingOptions:
    startup_model_path: Optional[str] = None
    startup_mmproj_path: Optional[str] = None
    default_backend: Optional[str] = "cpu"
    supported_backends: List[Dict[str, str]] = field(default_factory=list)
    default_web_max_tokens: int = DEFAULT_WEB_MAX_TOKENS
    max_text_file_chars: int = DEFAULT_MAX_TEXT_FILE_CHARS
    upload_directory: str = "uploads"
    log_directory: str = "logs"
    file_logging_enabled: bool = True
    default_sampling_config: SamplingConfig = field(default_factory=SamplingConfig)
    host: str = "127.0.0.1"
    port: int = 5000
    max_context: Optional[int] = None
    max_sessions: int = 1
    max_batch: int = 1                 # requests that run together (their model calls share steps)
    replicas: int = 1                  # server processes (one per GPU) behind the one address
    parallel: str = "tp"               # layout of a model started under torch.distributed.run: tp, pp or cp
    web_root: Optional[str] = None

    @property
    def supported_backend_values(self):
        return {b["value"].lower() for b in self.supported_backends}


def _read_option(args: Sequence[str], i: int, option: str) -> Tuple[Optional[str], int, bool]:
    a = args[i]
    if a.lower() == option:
        if i + 1 >= len(args):
            raise ValueError(f"Missing value for option '{option}'.")
        return args[i + 1], i + 1, True
    if a.lower().startswith(option + "="):
        return a[len(option) + 1:], i, True
    return None, i, False


def _pos_int(s: Optional[str]) -> Optional[int]:
    try:
        v = int(s.strip()) if s is not None else 0
    except ValueError:
        return None
    return v if v > 0 else None


def _listener_from_urls(urls: Optional[str]):
    """Host and port of the first ``http://`` entry of an ``ASPNETCORE_URLS`` value (``http://0.0.0.0:8080;...``), the
    listener setting the reference's host process reads; ``(None, None)`` when there is none.  ``*`` and ``+`` mean
    every interface."""
    for part in (urls or "").split(";"):
        part = part.strip()
        if not part.lower().startswith("http://"):
            continue
        rest = part[7:].split("/", 1)[0]
        host, _, port = rest.rpartition(":") if ":" in rest and not rest.endswith("]") else (rest, "", "")
        host = host.strip("[]")
        if host in ("*", "+", ""):
            host = "0.0.0.0"
        return host, _pos_int(port) or 80
    return None, None


def _pfloat(flag: str, s: str) -> float:
    try:
        return float(s)
    except ValueError:
        raise ValueError(f"Invalid value for {flag}: '{s}'.") from None


def _pint(flag: str, s: str) -> int:
    try:
        return int(s)
    except ValueError:
        raise ValueError(f"Invalid value for {flag}: '{s}'.") from None


_SAMPLING_FLAGS = (
    ("--temperature", "temperature", _pfloat, "TENSORSHARP_TEMPERATURE"),
    ("--top-k", "top_k", _pint, "TENSORSHARP_TOP_K"),
    ("--top-p", "top_p", _pfloat, "TENSORSHARP_TOP_P"),
    ("--min-p", "min_p", _pfloat, "TENSORSHARP_MIN_P"),
    ("--repeat-penalty", "repetition_penalty", _pfloat, "TENSORSHARP_REPEAT_PENALTY"),
    ("--presence-penalty", "presence_penalty", _pfloat, "TENSORSHARP_PRESENCE_PENALTY"),
    ("--frequency-penalty", "frequency_penalty", _pfloat, "TENSORSHARP_FREQUENCY_PENALTY"),
    ("--seed", "seed", _pint, "TENSORSHARP_SEED"),
)


def _parallel_layout(v) -> str:
    v = (str(v).strip().lower() if v else "tp")
    if v not in ("tp", "pp", "cp"):
        raise ValueError(f"--parallel must be tp, pp or cp, got '{v}'")
    return v


def parse_args(args: Sequence[str]) -> Dict[str, object]:
    out: Dict[str, object] = {"sampling": {}, "stop": None}
    plain = (("--model", "model"), ("--mmproj", "mmproj"), ("--backend", "backend"), ("--host", "host"),
             ("--parallel", "parallel"), ("--kv-dtype", "kv_dtype"))
    ints = (("--port", "port"), ("--max-context", "max_context"), ("--max-sessions", "max_sessions"),
            ("--max-batch", "max_batch"), ("--replicas", "replicas"))
    i = 0
    while i < len(args):
        matched = False
        for flag, key in plain:
            v, i, ok = _read_option(args, i, flag)
            if ok:
                out[key] = v
                matched = True
                break
        if not matched:
            v, i, ok = _read_option(args, i, "--max-tokens")
            if ok:
                p = _pos_int(v)
                if p is None:
                    raise ValueError(f"Invalid value for --max-tokens: '{v}'.")
                out["max_tokens"] = p
                matched = True
        if not matched:
            for flag, key in ints:
                v, i, ok = _read_option(args, i, flag)
                if ok:
                    out[key] = _pint(flag, v)
                    matched = True
                    break
        if not matched:
            for flag, key, conv, _env in _SAMPLING_FLAGS:
                v, i, ok = _read_option(args, i, flag)
                if ok:
                    out["sampling"][key] = conv(flag, v)
                    matched = True
                    break
        if not matched:
            v, i, ok = _read_option(args, i, "--stop")
            if ok:
                out["stop"] = (out["stop"] or []) + [v]
        i += 1
    return out


def resolve_default_sampling(overrides: Dict[str, object], stop: Optional[List[str]], env=None) -> SamplingConfig:
    env = os.environ if env is None else env
    cfg = SamplingConfig()
    for flag, key, conv, env_name in _SAMPLING_FLAGS:
        if key in overrides:
            setattr(cfg, key, overrides[key])
            continue
        raw = env.get(env_name)
        if raw is None or not raw.strip():
            continue
        try:
            setattr(cfg, key, conv(flag, raw.strip()))
        except ValueError:
            pass
    if stop is not None:
        cfg.stop_sequences = list(stop)
    return cfg


def resolve_mmproj_path(configured: Optional[str], model_path: Optional[str]) -> Optional[str]:
    if configured is None or not configured.strip() or configured.lower() == "none":
        return None
    if os.path.isabs(configured) or os.sep in configured or "/" in configured or os.path.exists(configured):
        return os.path.abspath(configured)
    d = os.path.dirname(model_path) if model_path else ""
    return os.path.abspath(os.path.join(d, configured)) if d else os.path.abspath(configured)


def build_options(args: Sequence[str], base_directory: str, env=None,
                  is_backend_available: Optional[Callable[[str], bool]] = None) -> ServerHostingOptions:
    if args is None:
        raise ValueError("args")
    if not base_directory:
        raise ValueError("base_directory")
    env = os.environ if env is None else env
    p = parse_args(args)
    model, mmproj = p.get("model"), p.get("mmproj")
    if mmproj and mmproj.strip() and not (model and model.strip()):
        raise ValueError("--mmproj requires --model.")
    model_path = os.path.abspath(model) if model and model.strip() else None
    mmproj_path = resolve_mmproj_path(mmproj, model_path)
    supported = supported_backends(is_backend_available)
    requested = p.get("backend") or env.get("BACKEND") or "b200"
    default_backend = resolve_default_backend(requested, supported)
    max_tokens = p.get("max_tokens") or _pos_int(env.get("MAX_TOKENS")) or DEFAULT_WEB_MAX_TOKENS
    max_text = _pos_int(env.get("MAX_TEXT_FILE_CHARS")) or DEFAULT_MAX_TEXT_FILE_CHARS
    upload_dir = os.path.join(base_directory, "uploads")
    os.makedirs(upload_dir, exist_ok=True)
    log_dir = env.get("TENSORSHARP_LOG_DIR")
    if not log_dir or not log_dir.strip():
        log_dir = os.path.join(base_directory, "logs")
    if p.get("kv_dtype"):
        # bf16 (default pages) or fp8 (e4m3 bytes): exported for ModelBase, which every model load of this process reads
        from ..cli.args import kv_dtype_name
        os.environ["TSB_KV_DTYPE"] = kv_dtype_name(str(p["kv_dtype"]))
    return ServerHostingOptions(
        startup_model_path=model_path, startup_mmproj_path=mmproj_path, default_backend=default_backend,
        supported_backends=supported, default_web_max_tokens=max_tokens, max_text_file_chars=max_text,
        upload_directory=upload_dir, log_directory=log_dir, file_logging_enabled=env.get("TENSORSHARP_LOG_FILE") != "0",
        default_sampling_config=resolve_default_sampling(p["sampling"], p["stop"], env),
        host=p.get("host") or env.get("TENSORSHARP_HOST") or _listener_from_urls(env.get("ASPNETCORE_URLS"))[0] or "127.0.0.1",
        port=int(p.get("port") or _pos_int(env.get("PORT")) or _listener_from_urls(env.get("ASPNETCORE_URLS"))[1] or 5000),
        max_context=p.get("max_context"), max_sessions=int(p.get("max_sessions") or 1),
        max_batch=int(p.get("max_batch") or _pos_int(env.get("TENSORSHARP_MAX_BATCH")) or 1),
        replicas=int(p.get("replicas") or _pos_int(env.get("TENSORSHARP_REPLICAS")) or 1),
        parallel=_parallel_layout(p.get("parallel") or env.get("TENSORSHARP_PARALLEL")))


def read_configured_backend_input(args: Sequence[str], env=None) -> Optional[str]:
    env = os.environ if env is None else env
    return parse_args(args).get("backend") or env.get("BACKEND")


# ---------------------------------------------------------------------------- backend selection
def try_resolve_supported_backend(options: ServerHostingOptions, requested: Optional[str]) -> Tuple[Optional[str], Optional[str]]:
    """Returns ``(backend, None)`` or ``(None, error)``."""
    resolved = options.default_backend if requested is None or not requested.strip() else canonicalize_backend(requested)
    if not resolved or resolved.lower() not in options.supported_backend_values:
        if not options.supported_backends:
            return None, "No supported backend is available on this machine."
        return None, f"Backend '{requested or options.default_backend}' is not supported on this machine."
    return resolved, None


# ---------------------------------------------------------------------------- hosted-model guard
def _stem(path: str) -> str:
    return os.path.splitext(os.path.basename(path))[0]


def matches_hosted_file_request(requested: Optional[str], hosted_path: Optional[str], allow_bare_model_id: bool) -> bool:
    if not requested or not requested.strip() or not hosted_path or not hosted_path.strip():
        return False
    t = requested.strip()
    if t.lower() == os.path.basename(hosted_path).lower():
        return True
    if allow_bare_model_id and t.lower() == _stem(hosted_path).lower():
        return True
    if os.sep in t or "/" in t or os.path.isabs(t):
        return os.path.abspath(t).lower() == os.path.abspath(hosted_path).lower()
    return False


def try_resolve_hosted_model_request(requested: Optional[str], hosted_path: Optional[str]) -> Tuple[Optional[str], Optional[str]]:
    if not hosted_path or not hosted_path.strip():
        return None, "No model is hosted by this server. Restart TensorSharp.Server with --model <path.gguf>."
    if not requested or not requested.strip():
        return None, "model is required"
    if not matches_hosted_file_request(requested, hosted_path, True):
        return None, (f"model '{requested}' is not hosted by this server. Restart TensorSharp.Server with "
                      "--model <path.gguf> to change it.")
    return hosted_path, None


def try_validate_hosted_mmproj_request(requested: Optional[str], hosted: Optional[str]) -> Optional[str]:
    """Returns ``None`` when acceptable, else the error text."""
    if requested is None:
        return None
    if not requested.strip() or requested.lower() == "none":
        if not hosted or not hosted.strip():
            return None
        return (f"This server was started with mmproj '{os.path.basename(hosted)}'. Restart TensorSharp.Server "
                "without --mmproj to host no projector.")
    if not hosted or not hosted.strip():
        return ("This server was started without --mmproj. Restart TensorSharp.Server with --mmproj <path.gguf> "
                "to host a projector.")
    if not matches_hosted_file_request(requested, hosted, False):
        return (f"mmproj '{requested}' is not hosted by this server. Restart TensorSharp.Server with "
                "--mmproj <path.gguf> to change it.")
    return None


def try_ensure_hosted_model_loaded(svc, requested: Optional[str], hosted_model: Optional[str],
                                   hosted_mmproj: Optional[str], backend: Optional[str]) -> Optional[str]:
    """Load the hosted model on first use; returns ``None`` on success, else the error text."""
    path, err = try_resolve_hosted_model_request(requested, hosted_model)
    if err:
        return err
    cb = canonicalize_backend(backend)
    if (svc.is_loaded and (svc.loaded_model_path or "").lower() == path.lower()
            and (svc.loaded_mmproj_path or "").lower() == (hosted_mmproj or "").lower()
            and (svc.loaded_backend or "").lower() == (cb or "").lower()):
        return None
    svc.load_model(path, hosted_mmproj, backend)
    if not svc.is_loaded:
        return f"Failed to load hosted model '{os.path.basename(path)}'."
    return None
