"""Interactive chat over ``.aio`` packages: archive loading, sampling, streaming display and the command loop
(reference ``loomchat.py:70-83,105-141,148-222,278-316,338-380,438-599``).  Generation runs on the decode engine:
the rendered conversation is prefilled in one fused pass and every further token is one CUDA-graph replay."""
from __future__ import annotations

import math
import os
import sys
import threading
from dataclasses import dataclass, fields
from typing import Dict, List, Optional, Tuple

import torch

from ..config import Config, resolve
from ..data.chat import ChatTemplate
from ..data.tokenizers import BPETokenizer, special_id
from ..models.loomformer import Model
from ..train import checkpoint as ckpt
from . import package as pk
from .decode import DecodeEngine

LOGO = "\n".join(("+------------------------------+", "| #       ###    ###   #   #   |", "| #      ##  #  ##  #  ## ##   |",
                  "| #      # # #  # # #  # # #   |", "| #   #  #  ##  #  ##  #   #   |", "| #####   ###    ###   #   #   |",
                  "+------------------------------+"))


class Paint:
    """ANSI styling that switches itself off when stdout is not a terminal or ``NO_COLOR`` is set."""
    CODES = dict(dim="2", bold="1", cyan="36", green="32", yellow="33", magenta="35", red="31", gray="90")

    def __init__(self, on: Optional[bool] = None) -> None:
        if on is None:
            on = sys.stdout.isatty() and not os.environ.get("NO_COLOR") and os.environ.get("TERM", "") != "dumb"
        self.on = bool(on)

    def __getattr__(self, name: str):
        code = Paint.CODES.get(name)
        if code is None:
            raise AttributeError(name)
        return (lambda s: f"\033[{code}m{s}\033[0m") if self.on else (lambda s: s)


PAINT = Paint()


@dataclass
class Settings:
    device: str
    dtype: str            # bf16 | fp16 | fp32
    temperature: float
    top_k: int
    top_p: float
    max_new: int
    window: int           # Tria temporal window (tokens between endpoint fires)
    alpha: float          # Tria carrier write strength
    beta: float           # PolARM correction strength

    def torch_dtype(self) -> torch.dtype:
        return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[self.dtype]


def default_dtype(device: torch.device) -> str:
    return "bf16" if device.type == "cuda" else "fp32"


class EscWatcher:
    """Background raw-key reader: pressing Esc sets ``requested``.  Inactive (never fires) when stdin is not a POSIX
    terminal, so piped input and tests behave as if nobody pressed anything."""

    def __init__(self) -> None:
        self.requested = threading.Event()
        self._halt = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._saved = None

    def __enter__(self) -> "EscWatcher":
        try:
            import termios, tty
            if sys.stdin.isatty():
                fd = sys.stdin.fileno()
                self._saved = (fd, termios.tcgetattr(fd))
                tty.setcbreak(fd)
                self._thread = threading.Thread(target=self._poll, daemon=True)
                self._thread.start()
        except Exception:
            self._saved = None
        return self

    def __exit__(self, *exc) -> None:
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=0.3)
        if self._saved is not None:
            import termios
            termios.tcsetattr(self._saved[0], termios.TCSADRAIN, self._saved[1])

    def _poll(self) -> None:
        import select
        fd = self._saved[0]
        while not self._halt.is_set():
            ready, _, _ = select.select([fd], [], [], 0.05)
            if ready and os.read(fd, 1) == b"\x1b":
                self.requested.set()
                return


def sample_next(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                generator: Optional[torch.Generator] = None) -> int:
    """One draw from 1-D logits: greedy at ``temperature <= 0``; otherwise temperature, then top-k truncation, then
    nucleus truncation (smallest sorted prefix whose mass reaches ``top_p``), all on the logits' device."""
    if temperature <= 0:
        return int(logits.argmax(-1))
    z = logits.float() / temperature
    if top_k and top_k > 0:
        kth = torch.topk(z, min(int(top_k), z.numel())).values[-1]
        z = z.masked_fill(z < kth, float("-inf"))
    p = torch.softmax(z, -1)
    if top_p and 0.0 < top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        keep = int(torch.searchsorted(sp.cumsum(-1), torch.tensor(float(top_p), device=sp.device))) + 1
        sp = sp[:keep]
        return int(si[torch.multinomial(sp / sp.sum(), 1, generator=generator)])
    return int(torch.multinomial(p, 1, generator=generator))


class StreamRenderer:
    """Prints only the new suffix of the turn decoded so far; ``<think>`` spans dimmed, ``<tool_call>`` spans held back
    until closed and then shown as one line."""

    def __init__(self, out=None) -> None:
        self.seen = ""
        self.thinking = False
        self.call: Optional[str] = None
        self.held = ""                     # tail that may be the beginning of a tag split across feeds
        self.out = out or sys.stdout

    TAGS = ("<tool_call>", "<think>", "</think>")

    def feed(self, text_so_far: str) -> None:
        new, self.seen = text_so_far[len(self.seen):], text_so_far
        if new:
            new, self.held = self.held + new, ""
            if self.call is None:
                for n in range(min(len(new), 10), 0, -1):
                    if any(t.startswith(new[-n:]) and t != new[-n:] for t in self.TAGS):
                        new, self.held = new[:-n], new[-n:]
                        break
            self._consume(new)

    def flush(self) -> None:
        tail, self.held = self.held, ""
        self._emit(tail)

    def _consume(self, s: str) -> None:
        while s:
            if self.call is not None:
                self.call += s
                if "</tool_call>" not in self.call:
                    return
                body, _, s = self.call.partition("</tool_call>")
                self.call = None
                print(PAINT.yellow(f"\n  → tool_call: {body.strip()}"), file=self.out, flush=True)
                continue
            tags = [(s.find(t), t) for t in ("<tool_call>", "</think>" if self.thinking else "<think>") if t in s]
            if not tags:
                self._emit(s)
                return
            at, tag = min(tags)
            self._emit(s[:at])
            s = s[at + len(tag):]
            if tag == "<tool_call>":
                self.call = ""
            else:
                self.thinking = tag == "<think>"

    def _emit(self, s: str) -> None:
        if s:
            print(PAINT.dim(s) if self.thinking else s, end="", file=self.out, flush=True)


class AIOChatTemplate(ChatTemplate):
    """Chat template whose Jinja source comes from the archive rather than a file."""

    def __init__(self, tok, source: str) -> None:
        super().__init__(tok, template_source=source)
        eos = special_id(tok, "<eos>")
        self.stop_ids = {i for i in (self.im_end_id, eos) if i is not None}


def archive_dtype(package: Dict) -> str:
    t = str(package.get("manifest", {}).get("quantization", {}).get("target_dtype", "none"))
    return t if t in ("bf16", "fp16", "fp32") else "fp32"


def load_aio(path: str, device: torch.device):
    """Returns ``(model, tokenizer, chat_template, cfg, manifest, packed_dtype)``."""
    if not str(path).lower().endswith(".aio"):
        raise ValueError("loomchat accepts only .aio archives")
    package = pk.load_aio(path)
    ck, tok_json, tpl = package.get("checkpoint"), package.get("tokenizer_json"), package.get("chat_template_jinja")
    if not isinstance(ck, dict):
        raise ValueError("AIO archive has no checkpoint")
    if not isinstance(tok_json, (bytes, bytearray)):
        raise ValueError("AIO archive has no tokenizer JSON")
    if not isinstance(tpl, (bytes, bytearray)):
        raise ValueError("AIO archive has no chat template")
    if ck.get("model_kind") != "loomformer":
        raise ValueError("AIO checkpoint is not a LoomFormer model")
    if ck.get("ffn_type") != "paraplex":
        raise ValueError("AIO checkpoint is not a Paraplex model")
    cfg = Config.from_checkpoint_dict(ck["cfg"])
    tok = BPETokenizer.from_json_bytes(bytes(tok_json))
    cfg.vocab = tok.vocab_size
    ablation = bool(ck.get("ablation", False))
    model = Model(cfg, ablation=ablation, dims=resolve(cfg, calibrate=False))
    model.carry_token_id = special_id(tok, "<CARRY>")
    ckpt.load_model_blob(model, ck, ablation)          # copies into fp32 storages; ties stay tied
    model.to(device).eval()
    return model, tok, AIOChatTemplate(tok, bytes(tpl).decode("utf-8")), cfg, package.get("manifest", {}), archive_dtype(package)


class ChatSession:
    """Model + decode engine + mutable settings.  Settings that the captured decode graph bakes in (window, alpha,
    beta, dtype, device) rebuild or invalidate the engine; sampler settings do not."""

    def __init__(self, aio_path: str, settings: Settings, dtype_override: Optional[str] = None) -> None:
        self.s = settings
        self.dtype_forced = dtype_override is not None
        self.engine: Optional[DecodeEngine] = None
        self.load(aio_path)

    def load(self, aio_path: str) -> None:
        dev = torch.device(self.s.device)
        self.model, self.tok, self.chat, self.cfg, self.manifest, packed = load_aio(aio_path, dev)
        if not self.dtype_forced:
            self.s.dtype = packed if dev.type == "cuda" else "fp32"
        self.s.window = self.s.window or int(self.cfg.tria_temporal_window or self.cfg.seq_len)
        self.cfg.tria_temporal_window = self.s.window
        self.s.alpha = float(self.cfg.tria_carrier_alpha)
        self.s.beta = float(self.cfg.tria_polarm_beta)
        self.path = aio_path
        self.engine = None

    def _engine(self) -> DecodeEngine:
        if self.engine is None:
            dev = torch.device(self.s.device)
            self.engine = DecodeEngine(self.model, batch=1, use_graph=(dev.type == "cuda"),
                                       dtype=self.s.torch_dtype() if dev.type == "cuda" else torch.float32)
        return self.engine

    def n_params(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    def set(self, name: str, value: str) -> Optional[str]:
        """Apply one setting; returns an error message or None."""
        s, cfg = self.s, self.cfg
        try:
            if name == "device":
                dev = torch.device(value)
                if dev.type == "cuda" and not torch.cuda.is_available():
                    return "CUDA is not available in this environment"
                self.model.to(dev)
                s.device, self.engine = value, None
            elif name == "dtype":
                if value not in ("bf16", "fp16", "fp32"):
                    return "dtype must be one of: bf16, fp16, fp32"
                s.dtype, self.engine, self.dtype_forced = value, None, True
            elif name == "window":
                w = int(value)
                if w <= 0:
                    return "window must be > 0"
                s.window = cfg.tria_temporal_window = w
            elif name == "alpha":
                a = float(value)
                if not math.isfinite(a) or a <= 0.0:
                    return "alpha must be finite and > 0"
                s.alpha = cfg.tria_carrier_alpha = a
            elif name == "beta":
                b = float(value)
                if not math.isfinite(b) or b < 0.0 or b >= 1.0:
                    return "beta must be finite and in [0, 1)"
                s.beta = cfg.tria_polarm_beta = b
            elif name == "temperature":
                s.temperature = float(value)
            elif name == "top_k":
                s.top_k = int(value)
            elif name == "top_p":
                s.top_p = float(value)
            elif name == "max_new":
                s.max_new = int(value)
            else:
                return f"unknown setting: {name}"
        except ValueError:
            return f"couldn't parse {value!r} for {name}"
        if name in ("window", "alpha", "beta") and self.engine is not None:
            self.engine.invalidate()
        return None

    @torch.no_grad()
    def generate_turn(self, messages: List[Dict], esc: Optional[EscWatcher] = None, out=None,
                      generator: Optional[torch.Generator] = None) -> Tuple[Dict, bool]:
        """Stream one assistant reply; returns ``(message, interrupted)``."""
        s = self.s
        ids = self.chat.render_prompt_ids(messages)
        seq_len = int(self.model.d.seq_len)
        room = seq_len - len(ids)
        if room <= 0:
            raise RuntimeError(f"conversation ({len(ids)} tokens) already fills the model's context (seq_len={seq_len}); "
                               "the incremental cache has no wraparound. /reset.")
        eng = self._engine()
        dev = torch.device(s.device)
        logits = eng.prefill(torch.tensor([ids], device=dev, dtype=torch.long))
        render = StreamRenderer(out)
        new: List[int] = []
        interrupted = False
        for _ in range(min(int(s.max_new), room)):
            if esc is not None and esc.requested.is_set():
                interrupted = True
                break
            nxt = sample_next(logits[0], s.temperature, s.top_k, s.top_p, generator)
            if nxt in self.chat.stop_ids:
                break
            new.append(nxt)
            render.feed(self.tok.decode(new, skip_special_tokens=False))
            logits = eng.step(torch.tensor([nxt], device=dev, dtype=torch.long))
        render.flush()
        print(file=out or sys.stdout)
        if interrupted:
            print(PAINT.gray("  (interrupted -- Esc)"), file=out or sys.stdout)
        raw = self.tok.decode(new, skip_special_tokens=False)
        calls = self.chat.parse_tool_calls(raw)
        if calls:
            return {"role": "assistant", "content": None, "tool_calls": calls}, interrupted
        return {"role": "assistant", "content": self.tok.decode(new, skip_special_tokens=True)}, interrupted


COMMANDS = {
    "/help": "show this list",
    "/settings": "show every current setting",
    "/device": "/device <cpu|cuda:0|cuda:1|...> -- move the model, reload nothing else",
    "/dtype": "/dtype <bf16|fp16|fp32>",
    "/window": "/window <int> -- Tria temporal window",
    "/alpha": "/alpha <float> -- Tria carrier write strength",
    "/beta": "/beta <float 0..1) -- PolARM correction strength",
    "/temperature": "/temperature <float>  (0 = greedy)",
    "/top-k": "/top-k <int>  (0 = disabled)",
    "/top-p": "/top-p <float 0..1>",
    "/max-new": "/max-new <int> -- cap on tokens generated per turn",
    "/system": "/system <text> -- set/replace the system prompt",
    "/reset": "clear conversation history (keeps the system prompt)",
    "/reload": "/reload <model.aio> -- swap archives without restarting",
    "/exit": "leave (also /quit)",
}
SETTING_COMMANDS = {"/device": "device", "/dtype": "dtype", "/window": "window", "/alpha": "alpha", "/beta": "beta",
                    "/temperature": "temperature", "/top-k": "top_k", "/top-p": "top_p", "/max-new": "max_new"}


def _menu(prefix: str) -> None:
    hits = [c for c in COMMANDS if c.startswith(prefix)]
    if hits:
        w = max(map(len, hits))
        print(PAINT.gray("  " + "   ".join(c.ljust(w) for c in hits)))


def handle_command(line: str, sess: ChatSession, messages: List[Dict]) -> Tuple[bool, bool]:
    """Process one ``/command`` line.  Returns ``(handled, leave)``."""
    if line == "/":
        _menu("")
        return True, False
    if line.startswith("/") and " " not in line and line not in ("/help", "/settings", "/reset", "/exit", "/quit"):
        hits = [c for c in COMMANDS if c.startswith(line)]
        if len(hits) != 1:
            _menu(line)
            return True, False
        line = hits[0]
    if line in ("/exit", "/quit"):
        return True, True
    if line == "/help":
        w = max(map(len, COMMANDS))
        for c, d in COMMANDS.items():
            print(f"  {PAINT.cyan(c.ljust(w))}  {PAINT.dim(d)}")
        return True, False
    if line == "/settings":
        for f in fields(sess.s):
            print(f"  {PAINT.cyan(f.name.ljust(12))} {getattr(sess.s, f.name)}")
        return True, False
    if line == "/reset":
        keep = messages[:1] if messages and messages[0]["role"] == "system" else []
        messages[:] = keep
        print(PAINT.dim("(history cleared)"))
        return True, False
    if line.startswith("/system "):
        msg = {"role": "system", "content": line[len("/system "):]}
        if messages and messages[0]["role"] == "system":
            messages[0] = msg
        else:
            messages.insert(0, msg)
        print(PAINT.dim("(system prompt set)"))
        return True, False
    if line.startswith("/reload "):
        target = line[len("/reload "):].strip()
        try:
            sess.s.window = 0
            sess.load(target)
            print(PAINT.dim(f"(reloaded {target})"))
        except Exception as e:   # keep the running session alive whatever the archive problem is
            print(PAINT.red(f"  ! reload failed: {e}"))
        return True, False
    for cmd, attr in SETTING_COMMANDS.items():
        if line.startswith(cmd + " "):
            err = sess.set(attr, line[len(cmd) + 1:].strip())
            print(PAINT.red(f"  ! {err}") if err else PAINT.dim(f"({attr}={getattr(sess.s, attr)})"))
            return True, False
    if line.startswith("/"):
        print(PAINT.red(f"  ! unknown command: {line}  (try /help)"))
        return True, False
    return False, False


def run_chat(aio_path: str, settings: Settings, system: Optional[str], dtype_override: Optional[str]) -> None:
    sess = ChatSession(aio_path, settings, dtype_override)
    quant = sess.manifest.get("quantization", {}).get("target_dtype", "none")
    print(PAINT.cyan(LOGO))
    print(PAINT.dim(f"  archive: {aio_path}  ({sess.n_params():,} params, packed={quant})"))
    print(PAINT.dim(f"  device={settings.device}  dtype={settings.dtype}  window={settings.window}  "
                    f"alpha={settings.alpha:g}  beta={settings.beta:g}"))
    print(PAINT.dim("  /help for commands · type / to browse them · Esc interrupts a reply\n"))
    messages: List[Dict] = [{"role": "system", "content": system}] if system else []
    while True:
        try:
            line = input(PAINT.bold(PAINT.green("you> "))).strip()
        except (EOFError, KeyboardInterrupt):
            print()
            return
        if not line:
            continue
        handled, leave = handle_command(line, sess, messages)
        if leave:
            return
        if handled:
            continue
        messages.append({"role": "user", "content": line})
        print(PAINT.bold(PAINT.magenta("loom> ")), end="", flush=True)
        try:
            with EscWatcher() as esc:
                reply, _ = sess.generate_turn(messages, esc)
        except RuntimeError as e:
            print(PAINT.red(f"\n  ! {e}"))
            messages.pop()
            continue
        messages.append(reply)
