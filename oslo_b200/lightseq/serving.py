"""A small HTTP inference server with dynamic batching around :func:`oslo_b200.lightseq.inference.generate`.

Counterpart of the serving back ends of the reference's LightSeq subset (oslo/lightseq2/inference/server,
inference/triton_backend: a Triton custom back end per model).  Triton is not part of this stack; the server here is a
FastAPI application:

* ``POST /generate``  ``{"input_ids": [[...]], "max_new_tokens": 32, "do_sample": false, ...}`` or ``{"text": "..."}`` when a
  tokenizer was given; answers ``{"output_ids": [[...]], "text": [...]?, "batched_with": n}``;
* ``GET /health``, ``GET /metrics`` (Prometheus text: requests, batches, batch-size histogram, latency);
* the inference protocol that Triton clients speak (KServe "v2" REST): ``GET /v2``, ``/v2/health/live``,
  ``/v2/health/ready``, ``/v2/models/{name}``, ``/v2/models/{name}/ready`` and ``POST /v2/models/{name}/infer`` with an
  ``input_ids`` INT64 tensor ``[batch, seq]`` (flat or nested ``data``) and generation settings under ``parameters``; the answer
  carries an ``output_ids`` INT64 tensor padded to the longest row.  So a client written against the reference's Triton
  back end needs a URL change only.

Requests wait in a queue; a single worker takes up to ``max_batch`` requests that arrive within ``max_wait_ms`` of the
first one and runs those with the same prompt length and sampling settings as one batch (prompts of other lengths in the
window run in their own batches: generation here takes no padding mask).  The model runs in a worker thread so the event
loop keeps accepting requests while the GPU is busy.
"""
from __future__ import annotations

import asyncio
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class _Request:
    input_ids: List[int]
    params: Dict[str, Any]
    future: "asyncio.Future" = field(repr=False, default=None)
    t0: float = 0.0


class DynamicBatcher:
    """Groups queued requests into batches and runs them through ``generate_fn(ids [b, s], **params) -> [b, s + new]``."""

    def __init__(self, generate_fn, max_batch: int = 8, max_wait_ms: float = 5.0):
        self.generate_fn, self.max_batch, self.max_wait = generate_fn, max_batch, max_wait_ms / 1000.0
        self.queue: "asyncio.Queue[_Request]" = None
        self.batches = self.requests = 0
        self.batch_sizes: List[int] = []
        self.latencies: List[float] = []
        self._task = None

    def start(self):
        if self.queue is None:
            self.queue = asyncio.Queue()
        if self._task is None or self._task.done():
            self._task = asyncio.get_running_loop().create_task(self._worker())

    async def stop(self):
        if self._task is not None:
            self._task.cancel()
            try:
                await self._task
            except asyncio.CancelledError:
                pass
            self._task = None

    async def submit(self, input_ids: List[int], **params):
        self.start()
        req = _Request(list(input_ids), params, asyncio.get_running_loop().create_future(), time.perf_counter())
        await self.queue.put(req)
        return await req.future

    async def _worker(self):
        while True:
            first = await self.queue.get()
            window = [first]
            deadline = time.perf_counter() + self.max_wait
            while len(window) < self.max_batch:
                left = deadline - time.perf_counter()
                if left <= 0:
                    break
                try:
                    window.append(await asyncio.wait_for(self.queue.get(), timeout=left))
                except asyncio.TimeoutError:
                    break
            groups: Dict[Any, List[_Request]] = {}
            for r in window:
                groups.setdefault((len(r.input_ids), tuple(sorted(r.params.items()))), []).append(r)
            for (_, _), reqs in groups.items():
                await self._run(reqs)

    async def _run(self, reqs: List[_Request]):
        ids = torch.tensor([r.input_ids for r in reqs], dtype=torch.long)
        try:
            out = await asyncio.get_running_loop().run_in_executor(None, lambda: self.generate_fn(ids, **reqs[0].params))
            rows = out.tolist()
            now = time.perf_counter()
            self.batches += 1
            self.requests += len(reqs)
            self.batch_sizes.append(len(reqs))
            for r, row in zip(reqs, rows):
                self.latencies.append(now - r.t0)
                if not r.future.done():
                    r.future.set_result((row, len(reqs)))
        except Exception as e:  # noqa: BLE001 - the error goes to every caller of the batch
            for r in reqs:
                if not r.future.done():
                    r.future.set_exception(e)


def create_app(model, tokenizer=None, device=None, max_batch: int = 8, max_wait_ms: float = 5.0, model_name: str = "oslo_b200",
               model_version: str = "1"):
    """Build the FastAPI application serving ``model`` (any causal LM accepted by ``generate``)."""
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import PlainTextResponse

    from .inference import generate

    device = device or next(model.parameters()).device
    allowed = {"max_new_tokens", "do_sample", "top_k", "top_p", "temperature", "num_beams", "no_repeat_ngram_size",
               "eos_token_id", "length_penalty"}

    def run(ids, **params):
        return generate(model, ids.to(device), **params).cpu()

    batcher = DynamicBatcher(run, max_batch, max_wait_ms)
    app = FastAPI(title="oslo_b200 inference")
    app.state.batcher = batcher

    @app.post("/generate")
    async def _generate(body: Dict[str, Any]):
        params = {k: v for k, v in body.items() if k in allowed}
        if "input_ids" in body:
            prompts = body["input_ids"]
            if prompts and isinstance(prompts[0], int):
                prompts = [prompts]
        elif "text" in body and tokenizer is not None:
            texts = body["text"] if isinstance(body["text"], list) else [body["text"]]
            prompts = [tokenizer(t)["input_ids"] for t in texts]
        else:
            raise HTTPException(status_code=422, detail="give input_ids (or text, when the server has a tokenizer)")
        if not prompts or any(len(p) == 0 for p in prompts):
            raise HTTPException(status_code=422, detail="empty prompt")
        try:
            results = await asyncio.gather(*[batcher.submit(p, **params) for p in prompts])
        except Exception as e:  # noqa: BLE001
            raise HTTPException(status_code=500, detail=repr(e))
        out = {"output_ids": [r[0] for r in results], "batched_with": [r[1] for r in results]}
        if tokenizer is not None and hasattr(tokenizer, "decode"):
            out["text"] = [tokenizer.decode(r[0]) for r in results]
        return out

    # ------------------------------------------------------------- KServe v2 ("Triton") protocol
    def _known(name: str, version: Optional[str] = None):
        if name != model_name or (version is not None and version != model_version):
            raise HTTPException(status_code=404, detail=f"unknown model {name!r}" + (f" version {version!r}" if version else ""))

    @app.get("/v2")
    async def _v2_server():
        return {"name": "oslo_b200", "version": model_version, "extensions": ["generate_parameters"]}

    @app.get("/v2/health/live")
    async def _v2_live():
        return {"live": True}

    @app.get("/v2/health/ready")
    async def _v2_ready():
        return {"ready": True}

    @app.get("/v2/models/{name}")
    async def _v2_model(name: str):
        _known(name)
        return {"name": model_name, "versions": [model_version], "platform": "oslo_b200",
                "inputs": [{"name": "input_ids", "datatype": "INT64", "shape": [-1, -1]}],
                "outputs": [{"name": "output_ids", "datatype": "INT64", "shape": [-1, -1]}]}

    @app.get("/v2/models/{name}/ready")
    async def _v2_model_ready(name: str):
        _known(name)
        return {"ready": True}

    async def _v2_infer_impl(name: str, body: Dict[str, Any], version: Optional[str] = None):
        _known(name, version)
        tensors = {t.get("name"): t for t in body.get("inputs", [])}
        t = tensors.get("input_ids")
        if t is None:
            raise HTTPException(status_code=400, detail="the request needs an input tensor named input_ids")
        if t.get("datatype", "INT64") not in ("INT64", "INT32"):
            raise HTTPException(status_code=400, detail="input_ids must be INT64 or INT32")
        shape, data = t.get("shape"), t.get("data")
        if not isinstance(shape, list) or len(shape) != 2 or data is None:
            raise HTTPException(status_code=400, detail="input_ids needs shape [batch, seq] and data")
        flat = [x for row in data for x in row] if data and isinstance(data[0], list) else list(data)
        b, sl = int(shape[0]), int(shape[1])
        if b <= 0 or sl <= 0 or len(flat) != b * sl:
            raise HTTPException(status_code=400, detail=f"data holds {len(flat)} elements, shape says {b} x {sl}")
        params = {k: v for k, v in (body.get("parameters") or {}).items() if k in allowed}
        pad = int((body.get("parameters") or {}).get("pad_token_id", 0))
        try:
            results = await asyncio.gather(*[batcher.submit([int(x) for x in flat[i * sl : (i + 1) * sl]], **params) for i in range(b)])
        except Exception as e:  # noqa: BLE001
            raise HTTPException(status_code=500, detail=repr(e))
        rows = [r[0] for r in results]
        width = max(len(r) for r in rows)
        out = [x for r in rows for x in (r + [pad] * (width - len(r)))]
        return {"model_name": model_name, "model_version": model_version, "id": body.get("id", ""),
                "outputs": [{"name": "output_ids", "datatype": "INT64", "shape": [b, width], "data": out}]}

    @app.post("/v2/models/{name}/infer")
    async def _v2_infer(name: str, body: Dict[str, Any]):
        return await _v2_infer_impl(name, body)

    @app.post("/v2/models/{name}/versions/{version}/infer")
    async def _v2_infer_version(name: str, version: str, body: Dict[str, Any]):
        return await _v2_infer_impl(name, body, version)

    @app.get("/health")
    async def _health():
        return {"status": "ok", "device": str(device), "requests": batcher.requests, "batches": batcher.batches}

    @app.get("/metrics", response_class=PlainTextResponse)
    async def _metrics():
        lat = sorted(batcher.latencies) or [0.0]
        lines = ["# TYPE oslo_requests_total counter", f"oslo_requests_total {batcher.requests}",
                 "# TYPE oslo_batches_total counter", f"oslo_batches_total {batcher.batches}",
                 "# TYPE oslo_batch_size_mean gauge",
                 f"oslo_batch_size_mean {sum(batcher.batch_sizes) / max(1, len(batcher.batch_sizes)):.3f}",
                 "# TYPE oslo_latency_seconds summary",
                 f'oslo_latency_seconds{{quantile="0.5"}} {lat[len(lat) // 2]:.6f}',
                 f'oslo_latency_seconds{{quantile="0.99"}} {lat[min(len(lat) - 1, int(len(lat) * 0.99))]:.6f}']
        return "\n".join(lines) + "\n"

    return app


def serve(model, host: str = "127.0.0.1", port: int = 8000, **kw):
    """Run the server with uvicorn (blocks)."""
    import uvicorn

    uvicorn.run(create_app(model, **kw), host=host, port=port)


__all__ = ["DynamicBatcher", "create_app", "serve"]
