"""HTTP serving layer: Ollama-, OpenAI- and web-UI-compatible endpoints over one hosted model.

Parity: TensorSharp.Server (Program.cs, Endpoints/*, ProtocolAdapters/*, ModelService.cs,
InferenceQueue.cs, SessionManager.cs).  The wire formats (routes, field names, field order,
which nulls are omitted, NDJSON / SSE framing) follow the reference; the engine underneath is
the paged-KV sm_100a runtime of this package.
"""
from .inference_queue import InferenceQueue, QueueTicket, QueueStatus
from .sessions import ChatSession, SessionManager
from .model_service import ModelService
from .options import ServerHostingOptions, build_options

__all__ = ["InferenceQueue", "QueueTicket", "QueueStatus", "ChatSession", "SessionManager", "ModelService",
           "ServerHostingOptions", "build_options"]
