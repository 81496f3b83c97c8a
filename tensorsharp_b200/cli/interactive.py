"""Interactive chat (REPL) with slash commands.

Parity: TensorSharp.Cli/InteractiveSession.cs — the command set of HandleCommand :266 (/help /exit
/reset /sampling /system /think /max /temp /topk /topp /minp /repeat /presence /frequency /seed
/stop /clearstop /image /audio /video /text /clearattach /multiline /save /history /model
/backend /mmproj /info and their aliases), attachments queued for the next turn, text files
inlined as ``[Attached file: name] ... [End of file]`` (ComposeUserContent :1036), multi-turn KV
reuse through the raw-token-splicing renderer, streaming through the architecture's output
parser, Ctrl+C cancels a running generation.
"""
from __future__ import annotations

import os
import signal
import time
from typing import Callable, List, Optional, Tuple

from ..runtime import media
from ..runtime.chat import ChatMessage, ToolFunction
from ..runtime.kv_cache import KVCache
from ..runtime.logging import Ev, NULL_LOGGER
from ..runtime.output_parser import create_output_parser
from ..runtime.prompt_renderer import GgufPromptRenderer, KVCachePromptRenderer
from ..runtime.sampling import SamplingConfig, TokenSampler

MAX_INLINED_TEXT_FILE_BYTES = 256 * 1024

HELP = """
Conversation:
  /help, /?              Show this message.
  /exit, /quit           Leave the session.
  /reset, /new           Clear conversation history and KV cache.
  /history               Print the current conversation history.
  /save <file>           Write the conversation transcript to a file.
  /savekv <file>         Write the cached tokens and KV rows (continue later without re-prefill).
  /loadkv <file>         Restore a KV state written by /savekv.
  /system <text>         Set (or clear when empty) the system prompt.
  /think on|off          Toggle thinking/reasoning mode for supported models.
  /multiline on|off      Toggle multi-line input (terminate with a single '.').

Model and runtime:
  /info, /status         Show the loaded model, backend, and projector.
  /model <path>          Load a different .gguf model (resets the session).
  /backend <name>        Reload the current model on a different backend (b200 | cpu).
  /mmproj <path>         Load a multimodal projector for the current model
                         (pass an empty value to clear).

Sampling:
  /sampling, /show       Print the current sampling configuration.
  /max <n>               Max tokens per reply.
  /temp <f>  /topk <n>  /topp <f>  /minp <f>
  /repeat <f>  /presence <f>  /frequency <f>  /seed <n>
  /stop <text>           Add a stop sequence.   /clearstop   Remove all stop sequences.

Attachments (queued for the next turn):
  /image <path>  /audio <path>  /video <path>  /text <path>
  /clearattach           Drop any pending image/audio/video/text attachments.

Plain text without a leading slash is sent to the model as the next user turn.
Press Ctrl+C while generating to interrupt; press Ctrl+C at the prompt to exit.
"""


def _parse_bool(s: str) -> Optional[bool]:
    v = s.strip().lower()
    if v in ("on", "true", "1", "yes", "y"):
        return True
    if v in ("off", "false", "0", "no", "n"):
        return False
    return None


def _strip_quotes(p: Optional[str]) -> str:
    p = (p or "").strip()
    if len(p) >= 2 and p[0] == p[-1] and p[0] in "\"'":
        return p[1:-1]
    return p


class InteractiveSession:
    def __init__(self, model, model_path: Optional[str], backend: str, mmproj_path: Optional[str], sampling: SamplingConfig,
                 tools: Optional[List[ToolFunction]], enable_thinking: bool, max_tokens: int, log=None, console=None,
                 read_line: Optional[Callable[[str], Optional[str]]] = None, model_loader=None):
        from .main import Console
        self.model, self.model_path, self.backend, self.mmproj_path = model, model_path, backend, mmproj_path
        self.sampling = sampling.clone()
        self.tools, self.think, self.max_tokens = tools, enable_thinking, max_tokens
        self.log = log or NULL_LOGGER
        self.con = console or Console()
        self._read = read_line or self._default_read
        self._load = model_loader
        self.renderer = KVCachePromptRenderer(GgufPromptRenderer())
        self.kv = KVCache()
        self.history: List[ChatMessage] = []
        self.system_prompt: Optional[str] = None
        self.multiline = False
        self.pending_images: List[str] = []
        self.pending_audios: List[str] = []
        self.pending_texts: List[Tuple[str, str]] = []
        self.pending_is_video = False
        self.should_exit = False
        self.generating = False
        self.cancel_requested = False

    # ------------------------------------------------------------------ I/O
    @staticmethod
    def _default_read(prompt: str) -> Optional[str]:
        try:
            return input(prompt)
        except EOFError:
            return None

    def say(self, text: str = "") -> None:
        self.con.print(text)

    def set_initial_system_prompt(self, text: str) -> None:
        self.system_prompt = text if text and text.strip() else None

    # ------------------------------------------------------------------ main loop
    def run(self) -> None:
        self.print_banner()
        old = None
        try:
            old = signal.signal(signal.SIGINT, self._on_sigint)
        except ValueError:                  # not the main thread (tests)
            pass
        try:
            while not self.should_exit:
                line = self._read_user_input()
                if line is None:
                    break
                if not line.strip():
                    continue
                if line.startswith("/"):
                    self.handle_command(line.strip())
                else:
                    self.run_turn(line)
        finally:
            if old is not None:
                signal.signal(signal.SIGINT, old)
        self.say("Bye.")

    def _on_sigint(self, signum, frame) -> None:
        if self.generating:
            self.cancel_requested = True
        else:
            raise KeyboardInterrupt

    def _read_user_input(self) -> Optional[str]:
        try:
            if not self.multiline:
                return self._read("\n>>> ")
            lines = []
            while True:
                l = self._read("... " if lines else "\n>>> ")
                if l is None:
                    return "\n".join(lines) if lines else None
                if not lines and l.startswith("/"):
                    return l
                if l.strip() == ".":
                    return "\n".join(lines)
                lines.append(l)
        except KeyboardInterrupt:
            return None

    def print_banner(self) -> None:
        from ..runtime.banner import render_banner
        out = getattr(self.con, "out", None)
        self.say(render_banner(["B200-native GGUF inference"], stream=out))
        self.say(f"TensorSharp B200 interactive chat - model {os.path.basename(self.model_path or '(unknown)')} "
                 f"[{self.model.arch}] on {self.backend}")
        self.say("Type /help for commands, /exit to quit.")
        self.print_sampling()

    def print_sampling(self, prefix: str = "") -> None:
        s = self.sampling
        stops = ", ".join('"%s"' % x for x in s.stop_sequences) if s.stop_sequences else "(none)"
        self.say(f"{prefix}Sampling: temperature={s.temperature:g} top_k={s.top_k} top_p={s.top_p:g} min_p={s.min_p:g} "
                 f"repeat_penalty={s.repetition_penalty:g} presence_penalty={s.presence_penalty:g} "
                 f"frequency_penalty={s.frequency_penalty:g} seed={s.seed} stop={stops} max_tokens={self.max_tokens} "
                 f"thinking={'on' if self.think else 'off'}")

    # ------------------------------------------------------------------ commands
    def handle_command(self, line: str) -> None:
        sp = line.find(" ")
        cmd, arg = (line, "") if sp < 0 else (line[:sp], line[sp + 1:].strip())
        cmd = cmd.lower()
        s = self.sampling
        table = {
            "/help": self.print_help, "/?": self.print_help,
            "/exit": self._exit, "/quit": self._exit,
            "/reset": self.reset_session, "/new": self.reset_session,
            "/sampling": self.print_sampling, "/show": self.print_sampling,
            "/clearstop": self.clear_stop_sequences, "/stop-clear": self.clear_stop_sequences,
            "/clearattach": self.clear_attachments, "/clear-attachments": self.clear_attachments,
            "/history": self.print_history, "/info": self.print_info, "/status": self.print_info,
        }
        with_arg = {
            "/system": self.set_system_prompt, "/think": self.set_thinking,
            "/max": self.set_max_tokens, "/maxtokens": self.set_max_tokens,
            "/seed": self.set_seed, "/stop": self.add_stop_sequence,
            "/image": self.attach_image, "/img": self.attach_image, "/audio": self.attach_audio,
            "/video": self.attach_video, "/vid": self.attach_video,
            "/text": self.attach_text_file, "/file": self.attach_text_file, "/txt": self.attach_text_file,
            "/multiline": self.toggle_multiline, "/save": self.save_transcript,
            "/model": self.load_different_model, "/backend": self.switch_backend,
            "/mmproj": self.load_mmproj, "/projector": self.load_mmproj,
            "/savekv": self.save_kv_state, "/loadkv": self.load_kv_state,
        }
        sampling = {
            ("/temp", "/temperature"): ("temperature", False), ("/topk", "/top-k", "/top_k"): ("top_k", True),
            ("/topp", "/top-p", "/top_p"): ("top_p", False), ("/minp", "/min-p", "/min_p"): ("min_p", False),
            ("/repeat", "/repeat-penalty", "/repetition-penalty"): ("repetition_penalty", False),
            ("/presence", "/presence-penalty"): ("presence_penalty", False),
            ("/frequency", "/frequency-penalty"): ("frequency_penalty", False),
        }
        if cmd in table:
            table[cmd]()
            return
        if cmd in with_arg:
            with_arg[cmd](arg)
            return
        for names, (attr, is_int) in sampling.items():
            if cmd in names:
                self.update_sampling(arg, attr, is_int)
                return
        self.say(f"Unknown command: {cmd}. Type /help for the list.")

    def print_help(self) -> None:
        self.say(HELP)

    def _exit(self) -> None:
        self.should_exit = True

    def reset_session(self) -> None:
        self.history.clear()
        self.kv.reset()
        self.model.reset_kv_cache()
        self.clear_attachments(quiet=True)
        self.say("Conversation history and KV cache cleared.")

    def set_system_prompt(self, text: str) -> None:
        self.system_prompt = text if text and text.strip() else None
        self.history.clear()
        self.kv.reset()
        self.model.reset_kv_cache()
        self.say("System prompt cleared. Conversation reset." if self.system_prompt is None
                 else f"System prompt set ({len(self.system_prompt)} chars). Conversation reset.")

    def set_thinking(self, arg: str) -> None:
        if not arg:
            self.think = not self.think
        else:
            v = _parse_bool(arg)
            if v is None:
                self.say(f"Could not parse '{arg}' as boolean. Use 'on' or 'off'.")
                return
            self.think = v
        self.say(f"Thinking is now {'on' if self.think else 'off'}.")

    def set_max_tokens(self, arg: str) -> None:
        try:
            v = int(arg)
            if v <= 0:
                raise ValueError
        except ValueError:
            self.say(f"Could not parse '{arg}' as a positive integer.")
            return
        self.max_tokens = v
        self.say(f"Max tokens per reply set to {v}.")

    def update_sampling(self, arg: str, attr: str, is_int: bool) -> None:
        if not arg:
            self.say(f"Usage: /{attr.replace('_', '-')} <{'int' if is_int else 'float'}>")
            return
        try:
            setattr(self.sampling, attr, int(arg) if is_int else float(arg))
        except ValueError:
            self.say(f"Could not parse '{arg}' as {'int' if is_int else 'float'} for {attr}.")
            return
        self.say(f"{attr} updated.")
        self.print_sampling()

    def set_seed(self, arg: str) -> None:
        try:
            v = int(arg)
        except ValueError:
            self.say(f"Could not parse '{arg}' as int for seed.")
            return
        self.sampling.seed = v
        self.say(f"Seed set to {v} ({'deterministic' if v >= 0 else 'random'}).")

    def add_stop_sequence(self, text: str) -> None:
        if not text:
            self.say("Usage: /stop <text>. Use /clearstop to remove all.")
            return
        self.sampling.stop_sequences = (self.sampling.stop_sequences or []) + [text]
        self.say(f'Added stop sequence "{text}". Now {len(self.sampling.stop_sequences)} configured.')

    def clear_stop_sequences(self) -> None:
        self.sampling.stop_sequences = None
        self.say("Cleared all stop sequences.")

    def attach_image(self, path: str) -> None:
        path = _strip_quotes(path)
        if not path or not os.path.isfile(path):
            self.say(f"Image file not found: {path}")
            return
        if self.pending_is_video:
            self.say("This turn already has a queued video. Use /clearattach before adding still images.")
            return
        self.pending_images.append(path)
        self.say(f"Image attached: {path}. {len(self.pending_images)} image(s) queued for next turn.")

    def attach_audio(self, path: str) -> None:
        path = _strip_quotes(path)
        if not path or not os.path.isfile(path):
            self.say(f"Audio file not found: {path}")
            return
        self.pending_audios.append(path)
        self.say(f"Audio attached: {path}. {len(self.pending_audios)} audio file(s) queued for next turn.")

    def attach_video(self, path: str) -> None:
        path = _strip_quotes(path)
        if not path or not os.path.isfile(path):
            self.say(f"Video file not found: {path}")
            return
        if self.pending_is_video:
            self.say("Another video is already queued for this turn. Use /clearattach to start over.")
            return
        if self.pending_images:
            self.say("Cannot attach a video when still images are already queued. Use /clearattach first.")
            return
        try:
            frames = media.extract_video_frames(path)
        except Exception as e:
            self.say(f"Failed to extract frames from video: {e}")
            return
        if not frames:
            self.say(f"No frames could be extracted from video: {path}")
            return
        self.pending_images.extend(frames)
        self.pending_is_video = True
        self.say(f"Video attached: {path}. Extracted {len(frames)} frame(s) for next turn.")

    def attach_text_file(self, path: str) -> None:
        path = _strip_quotes(path)
        if not path or not os.path.isfile(path):
            self.say(f"Text file not found: {path}")
            return
        try:
            size = os.path.getsize(path)
            with open(path, "rb") as f:
                data = f.read(MAX_INLINED_TEXT_FILE_BYTES)
            if size > MAX_INLINED_TEXT_FILE_BYTES:
                self.say(f"Text file is {size} bytes; only the first {MAX_INLINED_TEXT_FILE_BYTES} bytes will be inlined.")
            content = data.decode("utf-8", errors="replace")
        except OSError as e:
            self.say(f"Failed to read text file: {e}")
            return
        self.pending_texts.append((path, content))
        self.say(f"Text file attached: {path} ({len(content)} chars). {len(self.pending_texts)} text file(s) queued for next turn.")

    def clear_attachments(self, quiet: bool = False) -> None:
        total = len(self.pending_images) + len(self.pending_audios) + len(self.pending_texts)
        self.pending_images.clear()
        self.pending_audios.clear()
        self.pending_texts.clear()
        self.pending_is_video = False
        if not quiet:
            self.say(f"Dropped {total} pending attachment(s)." if total else "No pending attachments.")

    def toggle_multiline(self, arg: str) -> None:
        if not arg:
            self.multiline = not self.multiline
        else:
            v = _parse_bool(arg)
            if v is None:
                self.say(f"Could not parse '{arg}' as boolean. Use 'on' or 'off'.")
                return
            self.multiline = v
        self.say("Multi-line input on: finish a message with a single '.' on its own line." if self.multiline
                 else "Multi-line input off.")

    def save_transcript(self, path: str) -> None:
        if not path:
            self.say("Usage: /save <file-path>")
            return
        try:
            with open(path, "w", encoding="utf-8") as w:
                if self.system_prompt:
                    w.write("=== System ===\n" + self.system_prompt + "\n")
                for m in self.history:
                    w.write(f"=== {m.role} ===\n")
                    if m.thinking:
                        w.write("[thinking]\n" + m.thinking + "\n[/thinking]\n")
                    w.write((m.content or "") + "\n")
            self.say(f"Transcript saved to {path} ({len(self.history)} message(s)).")
        except OSError as e:
            self.say(f"Failed to save transcript: {e}")

    def save_kv_state(self, path: str) -> None:
        """Write the cached tokens and their K / V rows so a later run can continue without re-prefill."""
        if not path:
            self.say("Usage: /savekv <file-path>")
            return
        from ..runtime.session_store import save_session
        try:
            n = save_session(path, self.model, self.kv)
            self.say(f"KV state saved to {path} ({n} token(s)).")
        except (OSError, RuntimeError) as e:
            self.say(f"Failed to save KV state: {e}")

    def load_kv_state(self, path: str) -> None:
        if not path:
            self.say("Usage: /loadkv <file-path>")
            return
        from ..runtime.session_store import load_session
        try:
            n = load_session(path, self.model, self.kv)
            self.say(f"KV state loaded from {path} ({n} token(s)); a prompt that starts with the same tokens reuses it.")
        except (OSError, RuntimeError, ValueError, KeyError) as e:
            self.say(f"Failed to load KV state: {e}")

    def print_history(self) -> None:
        if not self.history and not self.system_prompt:
            self.say("(no conversation yet)")
            return
        self.say()
        if self.system_prompt:
            self.say("--- system ---\n" + self.system_prompt)
        for m in self.history:
            self.say(f"--- {m.role} ---")
            if m.thinking:
                self.say("[thinking]\n" + m.thinking + "\n[/thinking]")
            self.say(m.content or "")

    def print_info(self) -> None:
        m = self.model
        mm = getattr(m, "multimodal", None)
        self.say("\n--- Loaded model ---")
        self.say(f"  Path:         {self.model_path or '(unknown)'}")
        self.say(f"  Backend:      {self.backend}")
        self.say(f"  Architecture: {m.arch or '(unknown)'}")
        self.say(f"  Context:      {m.max_context} tokens (current KV: {getattr(m, 'cache_length', 0)})")
        self.say(f"  Vocab size:   {m.cfg.vocab}")
        self.say(f"  Projector:    {self.mmproj_path or '(none)'}")
        self.say(f"  Vision enc:   {'loaded' if mm is not None and getattr(mm, 'has_vision_encoder', False) else '(none)'}")
        turns = sum(1 for x in self.history if x.role == "user")
        self.say(f"  Conversation: {turns} user turn(s), KV cache holds {self.kv.count} token(s).")
        if self.pending_images or self.pending_audios or self.pending_texts:
            self.say(f"  Pending:      {len(self.pending_images)} image(s){' (video frames)' if self.pending_is_video else ''}, "
                     f"{len(self.pending_audios)} audio, {len(self.pending_texts)} text file(s).")

    # ------------------------------------------------------------------ model management
    def _reload(self, model_path: str, backend: str, mmproj: Optional[str], label: str) -> None:
        from .main import resolve_device
        loader = self._load
        if loader is None:
            from ..models.base import ModelBase
            loader = lambda p, b: ModelBase.create(p, resolve_device(b))   # noqa: E731
        self.say(f"{label}...")
        t0 = time.perf_counter()
        try:
            new_model = loader(model_path, backend)
        except Exception as e:
            self.say(f"Failed: {e}. Keeping the current model.")
            return
        self.model.close()
        self.model, self.model_path, self.backend = new_model, model_path, backend
        self.mmproj_path = None
        if mmproj:
            mm = getattr(new_model, "multimodal", None)
            if mm is None:
                self.say("This architecture has no multimodal encoder in this build; projector ignored.")
            else:
                mm.load_projectors(mmproj)
                self.mmproj_path = mmproj
        self.history.clear()
        self.kv.reset()
        self.clear_attachments(quiet=True)
        self.say(f"Loaded {os.path.basename(model_path)} [{new_model.arch}] on {backend} in {time.perf_counter() - t0:.1f}s. "
                 "Conversation reset.")

    def load_different_model(self, arg: str) -> None:
        path = _strip_quotes(arg)
        if not path or not os.path.isfile(path):
            self.say(f"Model file not found: {path}")
            return
        self._reload(path, self.backend, None, f"Loading {os.path.basename(path)}")

    def switch_backend(self, arg: str) -> None:
        from ..server.options import canonicalize_backend
        b = canonicalize_backend(arg)
        if b not in ("b200", "cpu"):
            self.say(f"Unknown backend '{arg}'. Use: b200, cpu.")
            return
        self._reload(self.model_path, b, self.mmproj_path, f"Reloading on {b}")

    def load_mmproj(self, arg: str) -> None:
        path = _strip_quotes(arg)
        mm = getattr(self.model, "multimodal", None)
        if not path:
            self.mmproj_path = None
            if mm is not None:
                mm.unload()
            self.say("Projector cleared.")
            return
        if not os.path.isfile(path):
            self.say(f"Projector file not found: {path}")
            return
        if mm is None:
            self.say("This architecture has no multimodal encoder in this build.")
            return
        mm.load_projectors(path)
        self.mmproj_path = path
        self.history.clear()
        self.kv.reset()
        self.model.reset_kv_cache()
        self.say(f"Projector loaded: {path}. Conversation reset.")

    # ------------------------------------------------------------------ turns
    def compose_user_content(self, text: str) -> str:
        if not self.pending_texts:
            return text or ""
        out = []
        for path, content in self.pending_texts:
            out.append(f"[Attached file: {os.path.basename(path)}]\n{content}")
            if not content.endswith("\n"):
                out.append("\n")
            out.append("[End of file]\n\n")
        out.append(text or "")
        return "".join(out)

    def build_render_history(self, text: str) -> List[ChatMessage]:
        self.history.append(ChatMessage(
            role="user", content=self.compose_user_content(text),
            image_paths=list(self.pending_images) or None, audio_paths=list(self.pending_audios) or None,
            text_file_paths=[p for p, _ in self.pending_texts] or None, is_video=self.pending_is_video))
        out = [ChatMessage(role="system", content=self.system_prompt)] if self.system_prompt else []
        return out + self.history

    def run_turn(self, text: str) -> None:
        render_history = self.build_render_history(text)
        self.generating, self.cancel_requested = True, False
        try:
            self.stream(render_history)
        except KeyboardInterrupt:
            self.say("\n[generation cancelled]")
        except Exception as e:
            self.say(f"\n[error] {e}")
            self.log.error(Ev.CliFailed, "Interactive turn failed: {Error}", exc=e, Error=str(e))
            if self.history and self.history[-1].role == "user":
                self.history.pop()
        finally:
            self.generating = False

    def stream(self, render_history: List[ChatMessage]) -> None:
        from .main import apply_reuse_plan
        model, arch = self.model, self.model.arch
        tokens = self.renderer.render_to_tokens(model.tokenizer, model.cfg.chat_template, render_history, arch, True,
                                                self.tools, self.think)
        mm = getattr(model, "multimodal", None)
        if mm is not None:
            tokens = mm.process_prompt_tokens(render_history, tokens)
        if len(tokens) + self.max_tokens > model.max_context:
            raise RuntimeError(f"Prompt ({len(tokens)} tokens) plus max tokens ({self.max_tokens}) exceeds the context "
                               f"({model.max_context}). Use /reset or lower /max.")
        self.clear_attachments(quiet=True)
        t0 = time.perf_counter()
        plan = self.kv.plan_reuse(tokens, model.supports_kv_truncation)
        if mm is not None:
            mm.queue_prompt_embeddings(plan.reused_prefix_length if plan.kind.value == "PartialReuse" else
                                       (len(tokens) if plan.kind.value == "ExactMatch" else 0))
        logits = apply_reuse_plan(model, self.kv, plan, tokens)
        prefill_s = time.perf_counter() - t0
        parser = create_output_parser(arch)
        parser.init(self.think, self.tools)
        sampler = TokenSampler(self.sampling)
        tok = model.tokenizer
        ids: List[int] = []
        raw = bytearray()
        emitted = 0
        content, thinking, tool_calls = [], [], None
        in_think = False
        t1 = time.perf_counter()

        def show(parsed) -> None:
            nonlocal in_think, tool_calls
            if parsed.thinking:
                if not in_think:
                    self.con.print("[thinking] ", end="")
                    in_think = True
                self.con.print(parsed.thinking, end="")
                thinking.append(parsed.thinking)
            if parsed.content:
                if in_think:
                    self.con.print("\n[/thinking]")
                    in_think = False
                self.con.print(parsed.content, end="")
                content.append(parsed.content)
            if parsed.tool_calls is not None:
                tool_calls = parsed.tool_calls

        from ..server.model_service import find_valid_utf8_length
        for _ in range(self.max_tokens):
            if self.cancel_requested:
                self.con.print("\n[generation cancelled]")
                break
            nxt = sampler.sample(logits, ids)
            if tok.is_eos(nxt):
                break
            ids.append(nxt)
            raw += tok.token_bytes(nxt)
            text = bytes(raw[:find_valid_utf8_length(raw)]).decode("utf-8", errors="replace")
            piece, emitted = text[emitted:], len(text)
            stop = False
            if self.sampling.stop_sequences:
                _, stop = sampler.check_stop_sequences(text)
            if piece:
                show(parser.add(piece, False))
            if stop:
                break
            logits = model.forward([nxt])
            self.kv.record_append(nxt, logits)
        show(parser.add("", True))
        if in_think:
            self.con.print("\n[/thinking]")
        dt = time.perf_counter() - t1
        if tool_calls:
            self.con.print("\n--- Tool Calls ---")
            for tc in tool_calls:
                self.con.print(f"  {tc}")
        self.con.print()
        self.con.print(f"[{len(ids)} tokens, {len(ids) / dt if dt > 0 else 0:.1f} tok/s, prompt {len(tokens)} tokens "
                       f"({plan.kind.value}, prefill {prefill_s * 1e3:.0f} ms)]")
        self.history.append(ChatMessage(role="assistant", content="".join(content), thinking="".join(thinking) or None,
                                        tool_calls=tool_calls, raw_output_tokens=ids))
