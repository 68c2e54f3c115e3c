"""OpenAI-compatible HTTP front end of the generation engine.

External agents (tool-use loops, gym-style resource servers) drive rollouts through ``/v1/completions`` and
``/v1/chat/completions`` while the trainer keeps refitting the same engine; the reference exposes vLLM's server for this
purpose (nemo_rl/models/generation/vllm/vllm_worker_async.py, ``expose_http_server``). Beyond the OpenAI fields every
choice carries what an RL trainer needs to train on the sample without re-tokenising: ``prompt_token_ids``,
``token_ids`` and per-token ``logprobs`` of the sampled tokens.

Requests that arrive within ``batch_window_s`` of each other and share their sampling parameters are served by one
engine call (continuous batching happens inside the engine; this front end only forms the request set).
"""

from __future__ import annotations

import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

from .engine import SamplingParams


@dataclass
class _Pending:
    prompt: list[int]
    key: tuple
    done: threading.Event = field(default_factory=threading.Event)
    record: Any = None
    error: Optional[str] = None


class BatchingFrontend:
    """Collects requests from many threads and runs them through the engine. ``continuous`` (default): ONE engine loop stays
    open while requests keep arriving; a request with the sampling settings of the running loop joins it at the engine's next
    host visit and is answered the moment it finishes (asynchronous, sample-level serving: the role of the reference's
    async vLLM engine, nemo_rl/models/generation/vllm/vllm_worker_async.py). Without it requests run in closed groups."""

    def __init__(self, engine, batch_window_s: float = 0.005, max_batch: int = 512, continuous: bool = True):
        self.engine, self.window, self.max_batch = engine, batch_window_s, max_batch
        self.continuous = continuous
        self.stats = dict(loops=0, joined_running_loop=0, answered=0)
        self._q: list[_Pending] = []
        self._cv = threading.Condition()
        self._stop = False
        self._paused = threading.Event()   # set while the trainer owns the engine (refit, training phase)
        self._idle = threading.Event()
        self._idle.set()
        self._calls = 0
        self._thread = threading.Thread(target=self._run, daemon=True, name="rlb-http-batcher")
        self._thread.start()

    # -- ownership hand-over with the trainer
    def pause(self, timeout_s: float = 600.0) -> bool:
        """Stops taking new batches and waits for the one in flight; the engine may then be refitted."""
        self._paused.set()
        return self._idle.wait(timeout_s)

    def resume(self) -> None:
        self._paused.clear()
        with self._cv:
            self._cv.notify_all()

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._thread.join(5.0)

    def submit(self, prompt: list[int], sp: dict, timeout_s: float = 600.0):
        key = (float(sp.get("temperature", 1.0)), float(sp.get("top_p", 1.0)), int(sp.get("top_k") or 0),
               int(sp.get("max_new_tokens", 256)), tuple(sp.get("stop_token_ids") or ()), bool(sp.get("greedy", False)))
        p = _Pending(list(prompt), key)
        with self._cv:
            self._q.append(p)
            self._cv.notify_all()
        if not p.done.wait(timeout_s):
            raise TimeoutError("generation request timed out")
        if p.error:
            raise RuntimeError(p.error)
        return p.record

    def _run_continuous(self) -> None:
        """One open engine loop for all queued (and still arriving) requests that share the first one's sampling settings."""
        with self._cv:
            if not self._q:
                self._idle.set()
                return
            key = self._q[0].key
        t, tp, tk, mx, stops, greedy = key
        self._calls += 1
        self.stats["loops"] += 1
        sp = SamplingParams(temperature=t, top_p=tp, top_k=tk, max_new_tokens=mx, stop_token_ids=list(stops), greedy=greedy, seed=1013 * self._calls)
        in_flight: set = set()
        first = [True]

        def admit():
            if self._paused.is_set() or self._stop:     # the trainer wants the engine: let the running requests drain
                return []
            with self._cv:
                room = self.max_batch - len(in_flight)
                take = [p for p in self._q if p.key == key][: max(0, room)]
                taken = set(map(id, take))
                self._q = [p for p in self._q if id(p) not in taken]
            if not first[0]:
                self.stats["joined_running_loop"] += len(take)
            first[0] = False
            out = []
            for p in take:
                in_flight.add(id(p))
                self._uid = getattr(self, "_uid", 0) + 1
                out.append((p.prompt, mx, self._uid, p))
            return out

        def finished(r):
            p = getattr(r, "tag", None)
            if p is None:
                return
            if getattr(r, "error", None):
                p.error = r.error
            p.record = r
            in_flight.discard(id(p))
            self.stats["answered"] += 1
            p.done.set()

        eng = self.engine
        eng.admit_hook, eng.finish_hook = admit, finished
        try:
            eng.wake()
            eng.generate([], sp)
        except Exception as e:
            with self._cv:
                stuck = [p for p in self._q if p.key == key]
            for p in stuck:      # requests of this loop that never got an answer are told why
                p.error = f"{type(e).__name__}: {e}"
                p.done.set()
            with self._cv:
                self._q = [p for p in self._q if p.key != key]
        finally:
            eng.admit_hook = eng.finish_hook = None
            self._idle.set()

    def _run(self) -> None:
        while True:
            with self._cv:
                while not self._stop and (not self._q or self._paused.is_set()):
                    self._cv.wait(0.05)
                if self._stop:
                    for p in self._q:
                        p.error = "server shutting down"
                        p.done.set()
                    return
                self._idle.clear()
            time.sleep(self.window)  # let concurrent requests join this batch
            if self.continuous:
                self._run_continuous()
                continue
            with self._cv:
                key = self._q[0].key
                batch = [p for p in self._q if p.key == key][: self.max_batch]
                taken = set(map(id, batch))
                self._q = [p for p in self._q if id(p) not in taken]
            try:
                self._calls += 1
                t, tp, tk, mx, stops, greedy = key
                sp = SamplingParams(temperature=t, top_p=tp, top_k=tk, max_new_tokens=mx, stop_token_ids=list(stops), greedy=greedy,
                                    seed=1013 * self._calls)
                self.engine.wake()
                recs = self.engine.generate([p.prompt for p in batch], sp)
                for p, r in zip(batch, recs):
                    p.record = r
            except Exception as e:  # the waiting request threads report the failure to their clients
                for p in batch:
                    p.error = f"{type(e).__name__}: {e}"
            finally:
                for p in batch:
                    p.done.set()
                self._idle.set()


def _render_chat(tokenizer, messages: list[dict]) -> list[int]:
    out = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
    if isinstance(out, dict):
        out = out["input_ids"]
    return list(out)


def create_app(engine, tokenizer, model_name: str = "policy", frontend: Optional[BatchingFrontend] = None,
               default_max_tokens: int = 256):
    """Builds the FastAPI application. ``engine`` is a :class:`GenerationEngine`; ``tokenizer`` needs ``encode``,
    ``decode`` and (for chat) ``apply_chat_template``."""
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="rl_b200 generation server")
    fe = frontend or BatchingFrontend(engine)
    app.state.frontend = fe
    app.state.weight_version = 0

    def _sampling(body: dict) -> dict:
        stops = list(body.get("stop_token_ids") or [])
        eos = getattr(tokenizer, "eos_token_id", None)
        if not body.get("ignore_eos", False) and eos is not None and eos not in stops:
            stops.append(eos)
        temp = float(body.get("temperature", 1.0))
        return dict(temperature=temp if temp > 0 else 1.0, greedy=temp == 0, top_p=float(body.get("top_p", 1.0)),
                    top_k=int(body.get("top_k") or 0) if (body.get("top_k") or 0) > 0 else 0,
                    max_new_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or default_max_tokens),
                    stop_token_ids=stops)

    def _cut_stop_strings(text: str, stop) -> tuple[str, bool]:
        if not stop:
            return text, False
        stops = [stop] if isinstance(stop, str) else list(stop)
        cut = min((text.find(s) for s in stops if s in text), default=-1)
        return (text[:cut], True) if cut >= 0 else (text, False)

    def _run(prompts: list[list[int]], body: dict) -> list[dict]:
        n = int(body.get("n", 1))
        sp = _sampling(body)
        jobs = [p for p in prompts for _ in range(n)]
        results: list[Any] = [None] * len(jobs)
        errors: list[str] = []

        def one(i):
            try:
                results[i] = fe.submit(jobs[i], sp)
            except Exception as e:
                errors.append(str(e))

        threads = [threading.Thread(target=one, args=(i,)) for i in range(len(jobs))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise HTTPException(status_code=503, detail=errors[0])
        out = []
        for i, r in enumerate(results):
            text = tokenizer.decode(r.out_tokens, skip_special_tokens=True)
            text, cut = _cut_stop_strings(text, body.get("stop"))
            finish = "stop" if (cut or not r.truncated) else "length"
            out.append(dict(index=i, text=text, finish_reason=finish, prompt_token_ids=list(r.prompt), token_ids=list(r.out_tokens),
                            logprobs=dict(token_logprobs=[float(x) for x in r.out_logprobs],
                                          tokens=[tokenizer.decode([t]) for t in r.out_tokens]) if body.get("logprobs") else None))
        return out

    def _usage(choices):
        pt = sum(len(c["prompt_token_ids"]) for c in choices)
        ct = sum(len(c["token_ids"]) for c in choices)
        return dict(prompt_tokens=pt, completion_tokens=ct, total_tokens=pt + ct)

    @app.get("/health")
    def health():
        return {"status": "ok", "weight_version": app.state.weight_version}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "rl_b200"}]}

    @app.post("/tokenize")
    def tokenize(body: dict):
        if "messages" in body:
            ids = _render_chat(tokenizer, body["messages"])
        else:
            ids = list(tokenizer.encode(body.get("prompt", "")))
        return {"tokens": ids, "count": len(ids)}

    @app.post("/detokenize")
    def detokenize(body: dict):
        return {"prompt": tokenizer.decode(list(body.get("tokens") or []))}

    @app.post("/v1/completions")
    def completions(body: dict):
        p = body.get("prompt", "")
        if isinstance(p, str):
            prompts = [list(tokenizer.encode(p))]
        elif p and isinstance(p[0], int):
            prompts = [list(p)]                       # token-in
        elif p and isinstance(p[0], str):
            prompts = [list(tokenizer.encode(s)) for s in p]
        else:
            prompts = [list(x) for x in p]
        if not prompts or any(len(x) == 0 for x in prompts):
            raise HTTPException(status_code=400, detail="empty prompt")
        choices = _run(prompts, body)
        return dict(id="cmpl-" + uuid.uuid4().hex[:16], object="text_completion", created=int(time.time()), model=model_name,
                    choices=choices, usage=_usage(choices), weight_version=app.state.weight_version)

    @app.post("/v1/chat/completions")
    def chat(body: dict):
        msgs = body.get("messages") or []
        if not msgs:
            raise HTTPException(status_code=400, detail="no messages")
        choices = _run([_render_chat(tokenizer, msgs)], body)
        for c in choices:
            c["message"] = {"role": "assistant", "content": c.pop("text")}
        return dict(id="chatcmpl-" + uuid.uuid4().hex[:16], object="chat.completion", created=int(time.time()), model=model_name,
                    choices=choices, usage=_usage(choices), weight_version=app.state.weight_version)

    return app


class ServerHandle:
    """A uvicorn server running the app on a background thread (``base_url`` is what clients and routers dial)."""

    def __init__(self, app, host: str = "127.0.0.1", port: int = 0):
        import socket

        import uvicorn

        if port == 0:
            with socket.socket() as s:
                s.bind((host, 0))
                port = s.getsockname()[1]
        self.app, self.host, self.port = app, host, port
        self.base_url = f"http://{host}:{port}"
        self._server = uvicorn.Server(uvicorn.Config(app, host=host, port=port, log_level="warning", access_log=False))
        self._thread = threading.Thread(target=self._server.run, daemon=True, name="rlb-http-server")

    def start(self, timeout_s: float = 10.0) -> "ServerHandle":
        self._thread.start()
        t0 = time.time()
        while not self._server.started and time.time() - t0 < timeout_s:
            time.sleep(0.01)
        if not self._server.started:
            raise RuntimeError("HTTP server did not start")
        return self

    def stop(self) -> None:
        self._server.should_exit = True
        self._thread.join(5.0)
        fe = getattr(self.app.state, "frontend", None)
        if fe is not None:
            fe.close()

    # trainer-side hooks: stop serving while weights change, then publish the new version
    def begin_weight_update(self) -> bool:
        return self.app.state.frontend.pause()

    def end_weight_update(self, version: Optional[int] = None) -> None:
        self.app.state.weight_version = self.app.state.weight_version + 1 if version is None else int(version)
        self.app.state.frontend.resume()
