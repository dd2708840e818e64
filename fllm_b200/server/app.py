"""One HTTP port speaking the OpenAI, Anthropic, Ollama, llama.cpp, TGI and SGLang dialects.

Architecture (cf. rust/engine/src/server.rs:765-823, :926-1140): HTTP handlers run on the
asyncio loop; the engine step loop runs on ONE worker thread and is the only code that touches
the engine. Handlers talk to it through a command queue (submit / abort) and get tokens back
through per-request asyncio queues. An exception inside a step is contained: every in-flight
request fails with an error id, their sequences are dropped and the loop continues; three
consecutive failures stop the worker so a supervisor can restart the process. ``/health`` is
liveness, ``/ready`` additionally requires a fresh worker heartbeat and no drain in progress.
"""
from __future__ import annotations

import asyncio
import contextlib
import json
import queue
import threading
import time
import uuid
from typing import Any, AsyncIterator, Dict, List, Optional

import torch
from fastapi import FastAPI, HTTPException, Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .. import __version__
from ..runtime.request import SamplingParams
from ..tokenizer import render_chat
from ..utils.metrics import Metrics


class EngineWorker:
    """Owns the engine on a dedicated thread."""

    STALL_S = 30.0

    def __init__(self, engine, metrics: Metrics, controller=None):
        """controller: runtime.step_control.StepController when this process is the front end of a multi-rank
        model instance; admissions, aborts and every step are then announced to the other ranks first."""
        self.engine, self.metrics = engine, metrics
        self.controller = controller
        self.comm_failed = False
        self.cmds: "queue.Queue[tuple]" = queue.Queue()
        self.streams: Dict[str, tuple] = {}          # request id -> (loop, asyncio.Queue, t_submit, n_prompt)
        self.heartbeat = time.monotonic()
        self.draining = False
        self.consecutive_failures = 0
        self.stopped = threading.Event()
        self.inject_failure = 0                       # test hook: number of steps that raise
        self.thread = threading.Thread(target=self._run, name="fllm-engine", daemon=True)

    def start(self) -> None:
        self.thread.start()

    def stop(self) -> None:
        self.stopped.set()
        self.cmds.put(("wake",))
        self.thread.join(timeout=10)
        if self.controller is not None:
            self.controller.shutdown()              # followers leave their loop

    # called from the asyncio side
    def submit(self, loop, rid: str, prompt: List[int], params: SamplingParams) -> "asyncio.Queue":
        q: asyncio.Queue = asyncio.Queue()
        self.cmds.put(("submit", rid, prompt, params, loop, q))
        return q

    def abort(self, rid: str) -> None:
        self.cmds.put(("abort", rid))

    async def call(self, fn):
        """Run fn(engine) on the engine thread; fn returns (result, events) and the events (of other
        requests that advanced meanwhile) are delivered like those of a normal step."""
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        self.cmds.put(("call", fn, loop, fut))
        return await fut

    def adopt(self, loop, rid: str, n_prompt: int, fn) -> "asyncio.Queue":
        """Register a stream for `rid`, then run fn(engine) (which must create that request)."""
        q: asyncio.Queue = asyncio.Queue()
        self.cmds.put(("adopt", rid, n_prompt, fn, loop, q))
        return q

    def ready(self) -> bool:
        return (not self.draining and not self.stopped.is_set() and not self.comm_failed
                and time.monotonic() - self.heartbeat < self.STALL_S)

    def _emit(self, rid: str, item: dict, final: bool) -> None:
        ent = self.streams.get(rid)
        if ent is None:
            return
        loop, q = ent[0], ent[1]
        loop.call_soon_threadsafe(q.put_nowait, item)
        if final:
            self.streams.pop(rid, None)

    def _drain_cmds(self, block: bool) -> None:
        try:
            cmd = self.cmds.get(timeout=0.05) if block else self.cmds.get_nowait()
        except queue.Empty:
            return
        while True:
            if cmd[0] == "submit":
                _, rid, prompt, params, loop, q = cmd
                self.streams[rid] = (loop, q, time.monotonic(), len(prompt))
                try:
                    if self.comm_failed:
                        raise RuntimeError("the model's rank group is down")
                    if self.controller is not None:
                        self.controller.admit(rid, prompt, params)
                    else:
                        self.engine.add_request(prompt, params, request_id=rid)
                    self.metrics.inc("fllm_prompt_tokens_total", len(prompt))
                except Exception as e:                                   # validation errors
                    self._emit(rid, {"error": str(e), "status": 503 if self.comm_failed else 400}, True)
            elif cmd[0] == "abort":
                if self.controller is not None:
                    self.controller.abort(cmd[1])
                else:
                    self.engine.abort_request(cmd[1])
                self.streams.pop(cmd[1], None)
            elif cmd[0] in ("call", "adopt") and self.controller is not None:
                # closures cannot travel to the other ranks: these operations (beam search, embeddings,
                # disaggregated hand-over) are single-rank features
                err = RuntimeError("this operation is not available when one server drives several ranks")
                if cmd[0] == "call":
                    cmd[2].call_soon_threadsafe(cmd[3].set_exception, err)
                else:
                    self.streams[cmd[1]] = (cmd[4], cmd[5], time.monotonic(), cmd[2])
                    self._emit(cmd[1], {"error": str(err), "status": 501}, True)
            elif cmd[0] == "call":
                _, fn, loop, fut = cmd
                try:
                    result, events = fn(self.engine)
                    self._dispatch(events)
                    loop.call_soon_threadsafe(fut.set_result, result)
                except Exception as e:
                    loop.call_soon_threadsafe(fut.set_exception, e)
            elif cmd[0] == "adopt":
                _, rid, n_prompt, fn, loop, q = cmd
                self.streams[rid] = (loop, q, time.monotonic(), n_prompt)
                try:
                    fn(self.engine)
                except Exception as e:
                    self._emit(rid, {"error": str(e), "status": 400}, True)
            try:
                cmd = self.cmds.get_nowait()
            except queue.Empty:
                return

    def _dispatch(self, events) -> None:
        now = time.monotonic()
        for ev in events:
            ent = self.streams.get(ev.request_id)
            if ent is not None and ev.token_ids:
                self.metrics.inc("fllm_generation_tokens_total", len(ev.token_ids))
            if ev.finished:
                self.metrics.inc("fllm_requests_total")
                if ent is not None:
                    self.metrics.observe("fllm_e2e_request_latency_seconds", now - ent[2])
            self._emit(ev.request_id, {"tokens": ev.token_ids, "finished": ev.finished,
                                       "reason": ev.finish_reason, "error": ev.error,
                                       "embedding": ev.embedding, "logprobs": ev.logprobs,
                                       "top_logprobs": ev.top_logprobs}, ev.finished)

    def _group_down(self, e: Exception) -> None:
        """A control collective failed: the other ranks are gone or late. Every request in flight ends with
        503, nothing new is admitted, readiness turns false; the process stays up to say so."""
        self.comm_failed = True
        self.draining = True
        self.metrics.inc("fllm_comm_failures_total")
        for rid in list(self.streams):
            try:
                self.engine.abort_request(rid)
            except Exception:
                pass
            self._emit(rid, {"error": f"model rank group failed: {e}", "status": 503}, True)

    def _run(self) -> None:
        from ..comm.group import CommError
        eng = self.engine
        ctl = self.controller
        while not self.stopped.is_set():
            self.heartbeat = time.monotonic()
            self._drain_cmds(block=not eng.has_unfinished())
            if self.comm_failed:
                continue
            if not eng.has_unfinished():
                if ctl is not None:
                    try:
                        ctl.idle_tick()
                    except CommError as e:
                        self._group_down(e)
                continue
            try:
                if self.inject_failure > 0:
                    self.inject_failure -= 1
                    raise RuntimeError("injected step failure")
                events = ctl.step() if ctl is not None else eng.step()
                self.consecutive_failures = 0
            except CommError as e:
                self._group_down(e)
                continue
            except Exception as e:                                       # contain, fail in-flight, continue
                self.consecutive_failures += 1
                self.metrics.inc("fllm_worker_panics_total")
                err_id = uuid.uuid4().hex[:12]
                for rid in list(self.streams):
                    (ctl.abort if ctl is not None else eng.abort_request)(rid)     # followers drop them too
                    self._emit(rid, {"error": f"internal error {err_id}: {type(e).__name__}", "status": 500}, True)
                if self.consecutive_failures >= 3:
                    self.stopped.set()
                continue
            self._dispatch(events)
            bm = eng.blocks
            self.metrics.set("fllm_kv_cache_usage", bm.num_used() / max(bm.num_blocks, 1))
            self.metrics.set("fllm_requests_running", len(eng.scheduler.running))
            self.metrics.set("fllm_requests_waiting", len(eng.scheduler.waiting))
            self.metrics.set("fllm_prefix_cache_hits", bm.stats["prefix_hits"])


# ---------------------------------------------------------------------------- helpers
def _sampling_from(body: dict, default_max: int = 256, dialect: str = "openai") -> SamplingParams:
    g = body.get
    opts = body.get("options", {}) if dialect == "ollama" else {}
    pick = lambda *names, default=None: next((src[n] for src in (body, opts) for n in names if src.get(n) is not None), default)
    stop = pick("stop", "stop_sequences", default=[])
    if isinstance(stop, str):
        stop = [stop]
    sp = SamplingParams(
        temperature=float(pick("temperature", default=1.0 if dialect != "llamacpp" else 0.8)),
        top_p=float(pick("top_p", default=1.0)), top_k=int(pick("top_k", default=0) or 0),
        min_p=float(pick("min_p", default=0.0)),
        repetition_penalty=float(pick("repetition_penalty", "repeat_penalty", default=1.0)),
        presence_penalty=float(pick("presence_penalty", default=0.0)),
        frequency_penalty=float(pick("frequency_penalty", default=0.0)),
        seed=pick("seed"), max_tokens=int(pick("max_tokens", "max_completion_tokens", "num_predict", "n_predict",
                                               "max_new_tokens", default=default_max)),
        min_tokens=int(pick("min_tokens", default=0)), ignore_eos=bool(pick("ignore_eos", default=False)),
        stop_token_ids=tuple(pick("stop_token_ids", default=()) or ()), stop=tuple(stop or ()),
        logit_bias={int(k): float(v) for k, v in (g("logit_bias") or {}).items()} or None,
        allowed_token_ids=g("allowed_token_ids"), logprobs=g("logprobs") is not None and g("logprobs") is not False,
        # chat: logprobs true + top_logprobs N; completions: logprobs N
        top_logprobs=int(g("top_logprobs") or (g("logprobs") if isinstance(g("logprobs"), int) and not isinstance(g("logprobs"), bool) else 0)),
        priority=int(g("priority") or 0), timeout_s=g("timeout"), cache_salt=str(g("cache_salt") or ""),
        typical_p=float(pick("typical_p", "typ_p", default=1.0)),
        dry_multiplier=float(pick("dry_multiplier", default=0.0)), dry_base=float(pick("dry_base", default=1.75)),
        dry_allowed_length=int(pick("dry_allowed_length", default=2)),
        dry_penalty_last_n=int(pick("dry_penalty_last_n", default=1024)),
        mirostat_mode=int(pick("mirostat", "mirostat_mode", default=0) or 0),
        mirostat_tau=float(pick("mirostat_tau", default=5.0)), mirostat_eta=float(pick("mirostat_eta", default=0.1)))
    # banned sequences / DRY breakers given as token-id lists are taken as they are; strings are tokenised by the caller
    bw = pick("bad_words_ids", "bad_words")
    if bw:
        seqs = [[int(t) for t in (w if isinstance(w, (list, tuple)) else [w])] for w in bw if not isinstance(w, str)]
        sp.bad_words = [q for q in seqs if q] or None
    br = pick("dry_sequence_breakers")
    if br:
        sp.dry_sequence_breakers = tuple(int(t) for t in br if not isinstance(t, str))
    if sp.max_tokens < 1:
        sp.max_tokens = default_max
    return sp


class StopChecker:
    """Incremental detokenisation with stop strings (text is held back while it could still
    turn into a stop sequence)."""

    def __init__(self, tokenizer, stops):
        self.tk, self.stops = tokenizer, [s for s in stops if s]
        self.ids: List[int] = []
        self.sent = 0
        self.hit = False

    def push(self, tokens: List[int], final: bool) -> str:
        self.ids.extend(tokens)
        text = self.tk.decode(self.ids)
        if text.endswith("�") and not final:        # incomplete UTF-8 sequence: wait
            text = text[:-1]
        for s in self.stops:
            i = text.find(s, max(0, self.sent - len(s)))
            if i >= 0:
                self.hit = True
                out = text[self.sent:i]
                self.sent = i
                return out
        hold = 0 if final else max((len(s) - 1 for s in self.stops), default=0)
        end = max(self.sent, len(text) - hold)
        out = text[self.sent:end]
        self.sent = end
        return out


GUIDED_KEYS = ("tools", "tool_choice", "guided_choice", "guided_regex", "guided_grammar", "grammar", "response_format",
               "format", "guided_json")


def make_guided_builder(engine, tokenizer, tool_parser):
    """-> build(body) giving the grammar object of a request (or None): forced tool calls, guided_choice, regular
    expressions, GBNF grammars, JSON mode and JSON schemas. Only the fields in GUIDED_KEYS are read, so the same
    fields rebuild the same recogniser on every rank of a tensor-parallel group. Raises ValueError on a bad grammar."""
    guided_shared: dict = {}

    def build(body: dict):
        tc = body.get("tool_choice")
        if body.get("tools") and tool_parser == "hermes" and (tc == "required" or (isinstance(tc, dict) and tc.get("function"))):
            # a forced tool call: the output is the call markup with one of the offered (or the named) functions
            from ..runtime.grammar import GuidedToolCall, TokenTrie
            if "trie" not in guided_shared:
                guided_shared["trie"] = TokenTrie.from_tokenizer(tokenizer)
                guided_shared["masks"] = {}
            names = ([tc["function"].get("name")] if isinstance(tc, dict)
                     else [(t.get("function") or {}).get("name") for t in body["tools"] if isinstance(t, dict)])
            eos = [getattr(tokenizer, "eos_token_id", None), getattr(engine, "eos_token_id", None)]
            try:
                return GuidedToolCall(guided_shared["trie"], tokenizer, eos, [n for n in names if n])
            except ValueError as e:
                raise ValueError(str(e))
        if body.get("guided_choice"):
            from ..runtime.grammar import GuidedChoice, TokenTrie
            if "trie" not in guided_shared:
                guided_shared["trie"] = TokenTrie.from_tokenizer(tokenizer)
                guided_shared["masks"] = {}
            eos = [getattr(tokenizer, "eos_token_id", None), getattr(engine, "eos_token_id", None)]
            try:
                return GuidedChoice(guided_shared["trie"], tokenizer, eos, body["guided_choice"])
            except (ValueError, TypeError) as e:
                raise ValueError(str(e))
        # general grammars: a regular expression, a GBNF grammar (vLLM's guided_regex / guided_grammar, llama.cpp's
        # grammar), or response_format {"type": "regex" | "grammar"}
        rf0 = body.get("response_format") if isinstance(body.get("response_format"), dict) else {}
        g_regex = body.get("guided_regex") or (rf0.get("pattern") if rf0.get("type") == "regex" else None)
        g_gbnf = body.get("guided_grammar") or body.get("grammar") or (rf0.get("grammar") if rf0.get("type") == "grammar" else None)
        if g_regex or g_gbnf:
            from ..runtime.grammar import TokenTrie
            from ..runtime.grammar_gbnf import GrammarError, GuidedGrammar, machine_from
            if "trie" not in guided_shared:
                guided_shared["trie"] = TokenTrie.from_tokenizer(tokenizer)
                guided_shared["masks"] = {}
            eos = [getattr(tokenizer, "eos_token_id", None), getattr(engine, "eos_token_id", None)]
            try:
                machine = machine_from("regex", str(g_regex)) if g_regex else machine_from("gbnf", str(g_gbnf))
            except (GrammarError, ValueError, IndexError) as e:
                raise ValueError(f"invalid grammar: {e}")
            return GuidedGrammar(guided_shared["trie"], tokenizer, eos, machine)
        rf = body.get("response_format")
        kind = rf.get("type") if isinstance(rf, dict) else None
        fmt = body.get("format")
        if kind not in ("json_object", "json_schema") and fmt != "json" and not isinstance(fmt, dict) \
                and not body.get("guided_json"):
            return None
        from ..runtime.grammar import GuidedJson, GuidedJsonSchema, TokenTrie
        if "trie" not in guided_shared:
            guided_shared["trie"] = TokenTrie.from_tokenizer(tokenizer)
            guided_shared["masks"] = {}
        eos = [getattr(tokenizer, "eos_token_id", None), getattr(engine, "eos_token_id", None)]
        schema = None
        if kind == "json_schema":
            js = rf.get("json_schema") or {}
            schema = js.get("schema") if isinstance(js.get("schema"), dict) else (js if "properties" in js else None)
        elif isinstance(body.get("guided_json"), dict):
            schema = body["guided_json"]
        elif isinstance(fmt, dict):
            schema = fmt
        if isinstance(schema, dict) and schema:
            # the whole schema (nested objects, arrays, enums, references ...) as a grammar; schemas that grammar
            # cannot express fall back to the recogniser that enforces the top-level object only
            from ..runtime.grammar_gbnf import GrammarError, GuidedGrammar, machine_from
            try:
                return GuidedGrammar(guided_shared["trie"], tokenizer, eos, machine_from("json_schema", schema))
            except (GrammarError, KeyError, TypeError, ValueError, IndexError, RecursionError):
                pass
        if isinstance(schema, dict) and schema.get("type", "object") == "object" and isinstance(schema.get("properties"), dict):
            try:
                return GuidedJsonSchema(guided_shared["trie"], tokenizer, eos, schema)
            except ValueError as e:
                raise ValueError(str(e))
        return GuidedJson(guided_shared["trie"], tokenizer, eos, require_object=True, cache=guided_shared["masks"])

    return build


def create_app(engine, tokenizer, model_name: str = "fllm-b200", api_key: Optional[str] = None,
               tool_parser: Optional[str] = None, reasoning_parser: Optional[str] = None,
               response_cache_entries: int = 256, response_cache_ttl_s: float = 600.0,
               otlp_endpoint: Optional[str] = None, controller=None, cors_origins: Optional[List[str]] = None,
               rate_limit_rps: float = 0.0) -> FastAPI:
    """controller: a runtime.step_control.StepController when this process fronts a multi-rank model instance
    (``serve --tp N`` on rank 0): every admission, abort and step is announced to the other ranks."""
    from .cache import ResponseCache, request_key
    from .parsers import REASONING_PARSERS, TOOL_PARSERS, ReasoningStream, parse_tool_calls, split_reasoning
    if tool_parser and tool_parser not in TOOL_PARSERS:
        raise ValueError(f"--tool-parser must be one of {TOOL_PARSERS}")
    if reasoning_parser and reasoning_parser not in REASONING_PARSERS:
        raise ValueError(f"--reasoning-parser must be one of {REASONING_PARSERS}")
    metrics = Metrics()
    worker = EngineWorker(engine, metrics, controller)
    rcache = ResponseCache(response_cache_entries, response_cache_ttl_s)
    from ..utils.telemetry import SpanExporter
    spans = SpanExporter(otlp_endpoint, service=model_name)
    guided_shared: dict = {}                     # token trie + mask cache, built on first use

    @contextlib.asynccontextmanager
    async def lifespan(_app):
        if not worker.thread.is_alive():
            worker.start()
        yield
        worker.stop()
        spans.shutdown()

    app = FastAPI(title="fllm_b200", version=__version__, lifespan=lifespan)
    app.state.worker, app.state.metrics, app.state.engine = worker, metrics, engine
    started = time.time()

    @app.middleware("http")
    async def _auth(request: HttpRequest, call_next):
        if api_key and request.url.path not in ("/health", "/ready", "/metrics", "/version"):
            tok = request.headers.get("authorization", "").removeprefix("Bearer ").strip() or \
                request.headers.get("x-api-key", "")
            if tok != api_key:
                return JSONResponse({"error": {"message": "invalid API key", "type": "authentication_error"}}, 401)
        return await call_next(request)

    # ------------------------------------------------------------------ core generation
    def encode_prompt(p) -> List[int]:
        if isinstance(p, list) and p and isinstance(p[0], int):
            return [int(t) for t in p]
        if isinstance(p, list) and p and isinstance(p[0], str):
            p = p[0]
        if not isinstance(p, str):
            raise HTTPException(400, "prompt must be a string or a list of token ids")
        return tokenizer.encode(p, add_bos=True)

    async def generate(prompt_ids: List[int], sp: SamplingParams, request: Optional[HttpRequest] = None) -> AsyncIterator[dict]:
        """Yields {"text", "tokens", "finished", "reason"} pieces."""
        if worker.draining:
            raise HTTPException(503, "server is draining")
        if worker.stopped.is_set():
            raise HTTPException(503, "engine worker stopped")
        try:
            sp.validate(engine.model_cfg.vocab_size)
        except ValueError as e:
            raise HTTPException(400, str(e))
        rid = "req-" + uuid.uuid4().hex
        q = worker.submit(asyncio.get_running_loop(), rid, prompt_ids, sp)
        chk = StopChecker(tokenizer, sp.stop)
        t0, first, last = time.monotonic(), True, None
        span = spans.start_span("llm.request", **{"request.id": rid, "llm.prompt_tokens": len(prompt_ids),
                                                  "llm.max_tokens": sp.max_tokens, "llm.temperature": float(sp.temperature)})
        n_out = 0
        try:
            while True:
                item = await q.get()
                if item.get("error"):
                    spans.end_span(span, ok=False, **{"error.message": str(item["error"])})
                    raise HTTPException(item.get("status", 500), item["error"])
                now = time.monotonic()
                n_out += len(item["tokens"])
                if item["tokens"]:
                    if first:
                        span.event("first_token")
                        metrics.observe("fllm_time_to_first_token_seconds", now - t0)
                        first = False
                    elif last is not None:
                        metrics.observe("fllm_inter_token_latency_seconds", (now - last) / max(len(item["tokens"]), 1))
                    last = now
                toks = [t for t in item["tokens"] if t != getattr(tokenizer, "eos_token_id", None) or sp.ignore_eos]
                text = chk.push(toks, item["finished"])
                if chk.hit and not item["finished"]:
                    worker.abort(rid)
                    spans.end_span(span, **{"llm.completion_tokens": n_out, "llm.finish_reason": "stop"})
                    yield {"text": text, "tokens": item["tokens"], "finished": True, "reason": "stop"}
                    return
                yield {"text": text, "tokens": item["tokens"], "finished": item["finished"],
                       "reason": "stop" if chk.hit else item["reason"], "embedding": item.get("embedding"),
                       "logprobs": item.get("logprobs"), "top_logprobs": item.get("top_logprobs")}
                if item["finished"]:
                    spans.end_span(span, **{"llm.completion_tokens": n_out, "llm.finish_reason": str(item["reason"])})
                    return
        except (asyncio.CancelledError, GeneratorExit):
            worker.abort(rid)
            spans.end_span(span, ok=False, **{"llm.completion_tokens": n_out, "llm.finish_reason": "cancelled"})
            raise

    async def collect(prompt_ids, sp):
        """Whole response of a non-streaming request; deterministic requests go through the
        response cache and identical requests in flight share one generation."""
        async def run():
            text, toks, reason = [], [], None
            async for piece in generate(prompt_ids, sp):
                text.append(piece["text"])
                toks.extend(piece["tokens"])
                reason = piece["reason"] or reason
            return "".join(text), toks, reason or "stop"
        return await rcache.get_or_compute(request_key(model_name, prompt_ids, sp), run)

    async def collect_with_logprobs(prompt_ids, sp):
        """Like `collect` for requests that ask for log-probabilities (never cached): also returns, per output
        token, its log-probability and the list of (token id, log-probability) alternatives."""
        text, toks, lps, tops, reason = [], [], [], [], None
        async for piece in generate(prompt_ids, sp):
            text.append(piece["text"])
            toks.extend(piece["tokens"])
            lps.extend(piece.get("logprobs") or [None] * len(piece["tokens"]))
            tops.extend(piece.get("top_logprobs") or [[] for _ in piece["tokens"]])
            reason = piece["reason"] or reason
        return "".join(text), toks, reason or "stop", lps, tops

    def piece_text(t: int) -> str:
        return tokenizer.decode([t])

    def chat_logprobs(toks, lps, tops) -> dict:
        def ent(t, lp):
            txt = piece_text(t)
            return {"token": txt, "logprob": lp, "bytes": list(txt.encode("utf-8", "replace"))}
        return {"content": [dict(ent(t, lp), top_logprobs=[ent(a, b) for a, b in alt]) for t, lp, alt in zip(toks, lps, tops)]}

    def completion_logprobs(toks, lps, tops) -> dict:
        texts = [piece_text(t) for t in toks]
        offs, o = [], 0
        for x in texts:
            offs.append(o)
            o += len(x)
        return {"tokens": texts, "token_logprobs": lps, "text_offset": offs,
                "top_logprobs": [{piece_text(a): b for a, b in alt} for alt in tops]}

    def choice_params(body: dict, default_max: int, first: SamplingParams) -> "List[SamplingParams]":
        """`n` choices are n requests: each with its own parameter object (a grammar state is per request) and,
        when a seed is given, seed + index so that the choices differ but the response repeats."""
        n = int(body.get("n") or 1)
        if not 1 <= n <= 16:
            raise HTTPException(400, "n must be in [1, 16]")
        out = [first]
        for i in range(1, n):
            spi = _sampling_from(body, default_max)
            attach_guided(spi, body)
            if spi.seed is not None:
                spi.seed = int(spi.seed) + i
            out.append(spi)
        return out

    build_guided = make_guided_builder(engine, tokenizer, tool_parser)

    def attach_guided(sp: SamplingParams, body: dict) -> None:
        """response_format json_object / json_schema (OpenAI) and format: "json" (Ollama) constrain the
        output to a JSON object through the sampler's allowed-token mask."""
        # banned words and DRY breakers given as text become token sequences (with and without a leading space)
        words = [w for w in (body.get("bad_words") or []) if isinstance(w, str) and w]
        if words:
            seqs = list(sp.bad_words or [])
            for w in words:
                for form in (w, " " + w):
                    ids = [int(t) for t in tokenizer.encode(form, add_bos=False)]
                    if ids and ids not in seqs:
                        seqs.append(ids)
            sp.bad_words = seqs
        brk = [w for w in (body.get("dry_sequence_breakers") or []) if isinstance(w, str) and w]
        if brk:
            extra = {int(tokenizer.encode(w, add_bos=False)[-1]) for w in brk if tokenizer.encode(w, add_bos=False)}
            sp.dry_sequence_breakers = tuple(sorted(set(sp.dry_sequence_breakers) | extra))
        try:
            g = build_guided(body)
        except ValueError as e:
            raise HTTPException(400, str(e))
        if g is not None:
            sp.guided = g
            sp.guided_spec = {k: body[k] for k in GUIDED_KEYS if k in body}

    def shape_message(text: str) -> "tuple[dict, bool]":
        """Assistant message of a finished chat turn: reasoning split off, tool calls parsed."""
        msg = {"role": "assistant"}
        if reasoning_parser:
            r, text = split_reasoning(text, reasoning_parser)
            if r:
                msg["reasoning_content"] = r
        calls = []
        if tool_parser:
            text, calls = parse_tool_calls(text, tool_parser)
        msg["content"] = text if (text or not calls) else None
        if calls:
            msg["tool_calls"] = calls
        return msg, bool(calls)

    def sse(gen) -> StreamingResponse:
        return StreamingResponse(gen, media_type="text/event-stream")

    # ------------------------------------------------------------------ health / admin
    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/ready")
    async def ready():
        if worker.ready():
            return {"status": "ready"}
        return JSONResponse({"status": "not ready", "draining": worker.draining}, 503)

    @app.get("/version")
    async def version():
        return {"version": __version__}

    @app.get("/metrics")
    async def prom():
        metrics.set("fllm_uptime_seconds", time.time() - started)
        metrics.set("fllm_draining", 1.0 if worker.draining else 0.0)
        return PlainTextResponse(metrics.render())

    @app.post("/admin/drain")
    async def drain(body: dict = {}):
        worker.draining = bool(body.get("enable", True)) if body else True
        return {"draining": worker.draining}

    @app.get("/admin/config")
    async def admin_config():
        from ..config import dump_effective
        return json.loads(dump_effective(engine.model_cfg, engine.cfg, engine.par))

    @app.get("/admin/prefix-cache")
    async def admin_prefix():
        return dict(engine.blocks.stats, cached_blocks=len(engine.blocks.cached), free_blocks=engine.blocks.num_free())

    @app.post("/admin/cache")
    async def admin_cache_reset():
        return {"freed_blocks": engine.blocks.reset_prefix_cache(), "dropped_responses": rcache.clear()}

    # disaggregated serving: a prefill server exports a processed prompt, a decode server adopts it
    def _pack_blob(blob: dict) -> dict:
        import base64
        kv = blob["kv"].contiguous()
        out = dict(blob)
        out["kv"] = {"shape": list(kv.shape), "elem": kv.element_size(),
                     "data": base64.b64encode(kv.view(torch.uint8).numpy().tobytes()).decode()}
        return out

    def _unpack_blob(obj: dict) -> dict:
        import base64
        kvd = obj["kv"]
        raw = torch.frombuffer(bytearray(base64.b64decode(kvd["data"])), dtype=torch.uint8)
        dt = engine.kv.store.dtype if kvd["elem"] == engine.kv.store.element_size() else None
        if dt is None:
            raise HTTPException(400, "KV element size does not match this engine")
        blob = dict(obj)
        blob["kv"] = raw.view(dt).view(*kvd["shape"])
        return blob

    @app.post("/admin/disagg/export")
    async def disagg_export(body: dict):
        """Process the prompt here and return the request (tokens + KV) for another server to decode."""
        ids = chat_prompt(body["messages"], body.get("tools")) if body.get("messages") else encode_prompt(body.get("prompt", ""))
        sp = _sampling_from(body, 256)
        try:
            blob = await worker.call(lambda eng: eng.prefill_only(ids, sp))
        except (ValueError, RuntimeError, KeyError) as e:
            raise HTTPException(400, str(e))
        return _pack_blob(blob)

    @app.post("/admin/disagg/import")
    async def disagg_import(body: dict):
        """Adopt an exported request and decode it to the end (non-streaming)."""
        blob = _unpack_blob(body)
        rid = "req-" + uuid.uuid4().hex
        q = worker.adopt(asyncio.get_running_loop(), rid, len(blob["prompt"]), lambda eng: eng.import_request(blob, rid))
        toks, reason = list(blob["output"]), None
        while True:
            item = await q.get()
            if item.get("error"):
                raise HTTPException(item.get("status", 500), item["error"])
            toks.extend(item["tokens"])
            if item["finished"]:
                reason = item["reason"]
                break
        eos = getattr(tokenizer, "eos_token_id", None)
        text = tokenizer.decode([t for t in toks if t != eos])
        return {"id": rid, "object": "text_completion", "model": model_name,
                "choices": [{"index": 0, "text": text, "token_ids": toks, "finish_reason": reason}],
                "usage": usage(len(blob["prompt"]), len(toks))}

    @app.get("/admin/telemetry")
    async def admin_telemetry():
        return spans.stats()

    @app.get("/admin/cache")
    async def admin_cache_stats():
        return {"responses": rcache.stats(), "prefix": dict(engine.blocks.stats)}

    @app.get("/admin/kv-tier")
    async def admin_kv_tier():
        t = getattr(engine, "kv_tier", None)
        return {"enabled": bool(t is not None and t.enabled), **(t.info() if t is not None else {}),
                "restored_blocks": engine.blocks.stats.get("tier_restored", 0)}

    # ------------------------------------------------------------------ OpenAI
    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": int(started),
                                            "owned_by": "fllm_b200", "max_model_len": engine.cfg.max_model_len}]}

    def usage(n_prompt, n_out):
        return {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}

    @app.post("/v1/completions")
    async def completions(body: dict):
        ids = encode_prompt(body.get("prompt", ""))
        sp = _sampling_from(body, 16)
        attach_guided(sp, body)
        cid = "cmpl-" + uuid.uuid4().hex
        if body.get("use_beam_search"):
            # beam search (non-streaming): `n` / `best_of` hypotheses, best first, with their length-normalised scores
            width = int(body.get("best_of") or body.get("n") or 4)
            try:
                def search(eng):
                    others: list = []
                    eos = -1 if sp.ignore_eos else getattr(tokenizer, "eos_token_id", None)     # -1: no token ends a hypothesis
                    return eng.beam_search(ids, width, sp.max_tokens, float(body.get("length_penalty", 1.0)), eos,
                                           bool(body.get("early_stopping", True)), others), others
                beams = await worker.call(search)
            except ValueError as e:
                raise HTTPException(400, str(e))
            eos_id = getattr(tokenizer, "eos_token_id", None)
            choices = []
            for i, (toks, score) in enumerate(beams[: int(body.get("n") or width)]):
                shown = [t for t in toks if t != eos_id]
                choices.append({"index": i, "text": tokenizer.decode(shown), "token_ids": toks, "logprobs": None,
                                "finish_reason": "stop" if toks and toks[-1] == eos_id else "length", "beam_score": score})
            return {"id": cid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                    "choices": choices, "usage": usage(len(ids), sum(len(c["token_ids"]) for c in choices))}
        if body.get("stream"):
            async def gen():
                async for piece in generate(ids, sp):
                    chunk = {"id": cid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                             "choices": [{"index": 0, "text": piece["text"], "token_ids": piece["tokens"],
                                          "finish_reason": piece["reason"] if piece["finished"] else None}]}
                    yield f"data: {json.dumps(chunk)}\n\n"
                yield "data: [DONE]\n\n"
            return sse(gen())
        async def one(spi, index):
            if spi.logprobs:
                text, toks, reason, lps, tops = await collect_with_logprobs(ids, spi)
                lp_obj = completion_logprobs(toks, lps, tops)
            else:
                (text, toks, reason), lp_obj = await collect(ids, spi), None
            return {"index": index, "text": text, "token_ids": toks, "finish_reason": reason, "logprobs": lp_obj}
        choices = await asyncio.gather(*[one(spi, i) for i, spi in enumerate(choice_params(body, 16, sp))])
        return {"id": cid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                "choices": list(choices), "usage": usage(len(ids), sum(len(c["token_ids"]) for c in choices))}

    def chat_prompt(messages, tools=None) -> List[int]:
        try:
            text = render_chat(getattr(tokenizer, "chat_template", None), messages, True, tools)
        except Exception as e:
            raise HTTPException(400, f"chat template error: {e}")
        return tokenizer.encode(text, add_bos=True)

    @app.post("/v1/chat/completions")
    async def chat_completions(body: dict):
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise HTTPException(400, "messages must be a non-empty list")
        ids = chat_prompt(msgs, body.get("tools"))
        sp = _sampling_from(body, 256)
        attach_guided(sp, body)
        cid = "chatcmpl-" + uuid.uuid4().hex
        if body.get("stream"):
            async def gen():
                head = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model_name,
                        "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]}
                yield f"data: {json.dumps(head)}\n\n"
                n = 0
                rs = ReasoningStream(reasoning_parser) if reasoning_parser else None
                held: List[str] = []                 # with a tool parser the text is held back and parsed at the end
                async for piece in generate(ids, sp):
                    n += len(piece["tokens"])
                    delta, fin = {}, piece["reason"] if piece["finished"] else None
                    text = piece["text"]
                    if rs is not None:
                        r, text = rs.push(text, piece["finished"])
                        if r:
                            delta["reasoning_content"] = r
                    if tool_parser:
                        held.append(text)
                        if piece["finished"]:
                            rest, calls = parse_tool_calls("".join(held), tool_parser)
                            if rest:
                                delta["content"] = rest
                            if calls:
                                delta["tool_calls"] = [dict(c, index=i) for i, c in enumerate(calls)]
                                fin = "tool_calls"
                    elif text:
                        delta["content"] = text
                    if not delta and not piece["finished"]:
                        continue
                    chunk = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model_name,
                             "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}
                    if piece["finished"] and (body.get("stream_options") or {}).get("include_usage"):
                        chunk["usage"] = usage(len(ids), n)
                    yield f"data: {json.dumps(chunk)}\n\n"
                yield "data: [DONE]\n\n"
            return sse(gen())
        async def one(spi, index):
            lp_obj = None
            if spi.logprobs:
                text, toks, reason, lps, tops = await collect_with_logprobs(ids, spi)
                lp_obj = chat_logprobs(toks, lps, tops)
            else:
                text, toks, reason = await collect(ids, spi)
            msg, has_calls = shape_message(text)
            choice = {"index": index, "message": msg, "finish_reason": "tool_calls" if has_calls else reason}
            if lp_obj is not None:
                choice["logprobs"] = lp_obj
            return choice, len(toks)
        done = await asyncio.gather(*[one(spi, i) for i, spi in enumerate(choice_params(body, 256, sp))])
        return {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": model_name,
                "choices": [c for c, _ in done], "usage": usage(len(ids), sum(n for _, n in done))}

    @app.post("/v1/chat/completions/render")
    async def chat_render(body: dict):
        ids = chat_prompt(body.get("messages", []), body.get("tools"))
        return {"prompt_token_ids": ids, "prompt": tokenizer.decode(ids)}

    async def embed_one(ids: List[int]) -> List[float]:
        """Decoder-as-encoder embedding: the final-norm hidden state of the last prompt token, L2-normalised."""
        sp = SamplingParams(max_tokens=1, temperature=0.0, embed=True, ignore_eos=True)
        vec = None
        async for piece in generate(ids, sp):
            vec = piece.get("embedding") or vec
        if vec is None:
            raise HTTPException(501, "this engine configuration cannot return hidden states")
        n = sum(v * v for v in vec) ** 0.5 or 1.0
        return [v / n for v in vec]

    def embedding_inputs(inp) -> List[List[int]]:
        if isinstance(inp, str):
            return [tokenizer.encode(inp, add_bos=True)]
        if isinstance(inp, list) and inp and all(isinstance(t, int) for t in inp):
            return [[int(t) for t in inp]]
        if isinstance(inp, list) and inp:
            return [encode_prompt(x) if not isinstance(x, str) else tokenizer.encode(x, add_bos=True) for x in inp]
        raise HTTPException(400, "input must be a string, a list of strings, or token ids")

    @app.post("/v1/embeddings")
    async def embeddings(body: dict):
        batches = embedding_inputs(body.get("input"))
        vecs = await asyncio.gather(*[embed_one(ids) for ids in batches])
        ntok = sum(len(b) for b in batches)
        return {"object": "list", "model": model_name,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/api/embed")
    async def ollama_embed(body: dict):
        batches = embedding_inputs(body.get("input"))
        return {"model": model_name, "embeddings": await asyncio.gather(*[embed_one(ids) for ids in batches])}

    @app.post("/api/embeddings")
    async def ollama_embeddings(body: dict):
        (ids,) = embedding_inputs(body.get("prompt", ""))[:1]
        return {"embedding": await embed_one(ids)}

    @app.post("/embedding")
    async def llamacpp_embedding(body: dict):
        (ids,) = embedding_inputs(body.get("content", ""))[:1]
        return {"embedding": await embed_one(ids)}

    # ------------------------------------------------------------------ Anthropic
    def anthropic_messages(body: dict) -> List[dict]:
        msgs = []
        sysm = body.get("system")
        if sysm:
            if isinstance(sysm, list):
                sysm = "".join(p.get("text", "") for p in sysm)
            msgs.append({"role": "system", "content": sysm})
        for m in body.get("messages", []):
            c = m.get("content")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if p.get("type") == "text")
            msgs.append({"role": m.get("role", "user"), "content": c})
        return msgs

    @app.post("/v1/messages")
    async def messages(body: dict):
        if "max_tokens" not in body:
            raise HTTPException(400, "max_tokens is required")
        ids = chat_prompt(anthropic_messages(body))
        sp = _sampling_from(body, 1024)
        mid = "msg_" + uuid.uuid4().hex
        stop_map = {"length": "max_tokens", "stop": "end_turn"}
        if body.get("stream"):
            async def gen():
                def ev(name, data):
                    return f"event: {name}\ndata: {json.dumps(data)}\n\n"
                yield ev("message_start", {"type": "message_start", "message": {
                    "id": mid, "type": "message", "role": "assistant", "content": [], "model": model_name,
                    "stop_reason": None, "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                yield ev("content_block_start", {"type": "content_block_start", "index": 0,
                                                 "content_block": {"type": "text", "text": ""}})
                n, reason = 0, "stop"
                async for piece in generate(ids, sp):
                    n += len(piece["tokens"])
                    if piece["text"]:
                        yield ev("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                         "delta": {"type": "text_delta", "text": piece["text"]}})
                    reason = piece["reason"] or reason
                yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": stop_map.get(reason, "end_turn")},
                                           "usage": {"output_tokens": n}})
                yield ev("message_stop", {"type": "message_stop"})
            return sse(gen())
        text, toks, reason = await collect(ids, sp)
        return {"id": mid, "type": "message", "role": "assistant", "model": model_name,
                "content": [{"type": "text", "text": text}], "stop_reason": stop_map.get(reason, "end_turn"),
                "stop_sequence": None, "usage": {"input_tokens": len(ids), "output_tokens": len(toks)}}

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(body: dict):
        return {"input_tokens": len(chat_prompt(anthropic_messages(body)))}

    # ------------------------------------------------------------------ Ollama
    @app.get("/api/version")
    async def ollama_version():
        return {"version": __version__}

    @app.get("/api/tags")
    async def ollama_tags():
        return {"models": [{"name": model_name, "model": model_name, "size": engine.weights.nbytes(),
                            "details": {"family": engine.model_cfg.arch, "parameter_size": f"{engine.model_cfg.param_count() / 1e9:.1f}B",
                                        "quantization_level": engine.model_cfg.weight_format}}]}

    @app.get("/api/ps")
    async def ollama_ps():
        return {"models": [{"name": model_name, "model": model_name, "size_vram": engine.weights.nbytes()}]}

    @app.post("/api/show")
    async def ollama_show(body: dict):
        return {"modelfile": "", "template": getattr(tokenizer, "chat_template", None) or "", "details": {
            "family": engine.model_cfg.arch}, "model_info": engine.model_cfg.to_dict()}

    def ollama_stream(ids, sp, make):
        async def gen():
            t0 = time.time()
            n = 0
            async for piece in generate(ids, sp):
                n += len(piece["tokens"])
                d = make(piece["text"], piece["finished"])
                if piece["finished"]:
                    d.update({"done_reason": piece["reason"], "prompt_eval_count": len(ids), "eval_count": n,
                              "total_duration": int((time.time() - t0) * 1e9)})
                yield json.dumps(d) + "\n"
        return StreamingResponse(gen(), media_type="application/x-ndjson")

    @app.post("/api/generate")
    async def ollama_generate(body: dict):
        ids = encode_prompt(body.get("prompt", "")) if body.get("raw") or not body.get("system") else \
            chat_prompt([{"role": "system", "content": body["system"]}, {"role": "user", "content": body.get("prompt", "")}])
        sp = _sampling_from(body, 128, "ollama")
        attach_guided(sp, body)
        now = lambda: time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
        if body.get("stream", True):
            return ollama_stream(ids, sp, lambda t, done: {"model": model_name, "created_at": now(), "response": t, "done": done})
        text, toks, reason = await collect(ids, sp)
        return {"model": model_name, "created_at": now(), "response": text, "done": True, "done_reason": reason,
                "prompt_eval_count": len(ids), "eval_count": len(toks)}

    @app.post("/api/chat")
    async def ollama_chat(body: dict):
        ids = chat_prompt(body.get("messages", []), body.get("tools"))
        sp = _sampling_from(body, 128, "ollama")
        attach_guided(sp, body)
        now = lambda: time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
        if body.get("stream", True):
            return ollama_stream(ids, sp, lambda t, done: {"model": model_name, "created_at": now(),
                                                           "message": {"role": "assistant", "content": t}, "done": done})
        text, toks, reason = await collect(ids, sp)
        return {"model": model_name, "created_at": now(), "message": {"role": "assistant", "content": text},
                "done": True, "done_reason": reason, "prompt_eval_count": len(ids), "eval_count": len(toks)}

    # ------------------------------------------------------------------ llama.cpp
    @app.post("/completion")
    async def llamacpp_completion(body: dict):
        ids = encode_prompt(body.get("prompt", ""))
        sp = _sampling_from(body, 128, "llamacpp")
        if body.get("stream"):
            async def gen():
                async for piece in generate(ids, sp):
                    yield f"data: {json.dumps({'content': piece['text'], 'stop': piece['finished']})}\n\n"
            return sse(gen())
        text, toks, reason = await collect(ids, sp)
        return {"content": text, "stop": True, "tokens_predicted": len(toks), "tokens_evaluated": len(ids),
                "stopped_limit": reason == "length", "stopped_eos": reason == "stop", "model": model_name}

    @app.post("/tokenize")
    async def tokenize(body: dict):
        return {"tokens": tokenizer.encode(body.get("content", ""), add_bos=bool(body.get("add_special")))}

    @app.post("/detokenize")
    async def detokenize(body: dict):
        return {"content": tokenizer.decode(body.get("tokens", []))}

    @app.get("/props")
    async def props():
        return {"model_path": model_name, "n_ctx": engine.cfg.max_model_len, "total_slots": engine.cfg.max_num_seqs,
                "chat_template": getattr(tokenizer, "chat_template", None) or ""}

    @app.get("/slots")
    async def slots():
        return [{"id": i, "is_processing": True, "n_decoded": len(r.output)} for i, r in enumerate(engine.scheduler.running)]

    @app.post("/apply-template")
    async def apply_template(body: dict):
        return {"prompt": render_chat(getattr(tokenizer, "chat_template", None), body.get("messages", []))}

    # ------------------------------------------------------------------ TGI / SGLang (shared /generate)
    @app.post("/generate")
    async def tgi_or_sglang_generate(body: dict):
        if "inputs" in body:                                   # TGI
            p = body.get("parameters", {}) or {}
            ids = encode_prompt(body["inputs"])
            sp = _sampling_from(p, 20)
            text, toks, reason = await collect(ids, sp)
            return {"generated_text": text, "details": {"finish_reason": "length" if reason == "length" else "eos_token",
                                                         "generated_tokens": len(toks)}}
        ids = body.get("input_ids") or encode_prompt(body.get("text", ""))     # SGLang
        sp = _sampling_from(body.get("sampling_params", {}) or {}, 128)
        text, toks, reason = await collect(ids, sp)
        return {"text": text, "meta_info": {"prompt_tokens": len(ids), "completion_tokens": len(toks),
                                            "finish_reason": {"type": reason}}}

    @app.post("/generate_stream")
    async def tgi_stream(body: dict):
        ids = encode_prompt(body.get("inputs", ""))
        sp = _sampling_from(body.get("parameters", {}) or {}, 20)

        async def gen():
            acc = []
            async for piece in generate(ids, sp):
                acc.append(piece["text"])
                d = {"token": {"id": piece["tokens"][-1] if piece["tokens"] else None, "text": piece["text"], "special": False},
                     "generated_text": "".join(acc) if piece["finished"] else None}
                yield f"data: {json.dumps(d)}\n\n"
        return sse(gen())

    @app.get("/info")
    async def tgi_info():
        return {"model_id": model_name, "max_total_tokens": engine.cfg.max_model_len, "version": __version__}

    @app.get("/get_model_info")
    async def sglang_model_info():
        return {"model_path": model_name, "is_generation": True}

    @app.get("/get_server_info")
    async def sglang_server_info():
        return {"version": __version__, "max_total_num_tokens": engine.blocks.num_blocks * engine.block_size}

    # Responses / Files / Batches, rerank / score / pooling / classify, infill, Ollama model management, CORS, rate limit
    from types import SimpleNamespace
    from . import extra_routes
    extra_routes.register(app, SimpleNamespace(
        engine=engine, worker=worker, tokenizer=tokenizer, model_name=model_name, started=started, generate=generate,
        collect=collect, embed_one=embed_one, encode_prompt=encode_prompt, chat_prompt=chat_prompt,
        sampling_from=_sampling_from, attach_guided=attach_guided, shape_message=shape_message, usage=usage, sse=sse))
    extra_routes.install_middleware(app, cors_origins, rate_limit_rps)
    return app


def serve(engine, tokenizer, host: str = "127.0.0.1", port: int = 8000, model_name: str = "fllm-b200",
          api_key: Optional[str] = None, log_level: str = "info", ssl_certfile: Optional[str] = None,
          ssl_keyfile: Optional[str] = None, **app_options) -> None:
    """ssl_certfile / ssl_keyfile: serve HTTPS (the reference's server/tls.rs)."""
    import uvicorn
    tls = {"ssl_certfile": ssl_certfile, "ssl_keyfile": ssl_keyfile} if ssl_certfile and ssl_keyfile else {}
    uvicorn.run(create_app(engine, tokenizer, model_name, api_key, **app_options), host=host, port=port,
                log_level=log_level, **tls)
