"""Web chat server: UI and streaming chat API from one FastAPI app, one model replica per GPU.

    python -m sample_efficient_gpt_b200.evals.chat_web --checkpoint /path/to/hf_dir --num-gpus 4

Endpoints and limits follow evals/chat_web.py:112-475 of the reference:
  GET /  (chat page)   POST /chat/completions (server-sent events)   GET /health   GET /stats
  at most 500 messages per request, 4000 characters per message, 8000 in total; temperature 0-2, top_k 1-200,
  max_tokens 1-2048; roles user|assistant.
Requests wait for a free replica (asyncio queue).  Tokens are streamed as they are sampled by this package's
``ChatEngine`` (``data: {"token": ..., "gpu": ...}`` lines, then ``data: {"done": true}``).
"""

from __future__ import annotations

import argparse
import asyncio
import json
import logging
from contextlib import asynccontextmanager
from dataclasses import dataclass

import torch
from fastapi import FastAPI, HTTPException
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import HTMLResponse, StreamingResponse
from pydantic import BaseModel

from sample_efficient_gpt_b200.evals.generation import ChatEngine, SamplingParams, load_engine

MAX_MESSAGES_PER_REQUEST = 500
MAX_MESSAGE_LENGTH = 4000
MAX_TOTAL_CONVERSATION_LENGTH = 8000
TEMPERATURE_RANGE = (0.0, 2.0)
TOP_K_RANGE = (1, 200)
MAX_TOKENS_RANGE = (1, 2048)

logger = logging.getLogger("chat_web")

PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>chat</title>
<style>body{font-family:sans-serif;max-width:760px;margin:2em auto}#log div{margin:.6em 0;white-space:pre-wrap}
.user{color:#024}.assistant{color:#040}textarea{width:100%;height:4em}</style></head><body>
<h3>Chat</h3><div id="log"></div><textarea id="box" placeholder="Message (Ctrl+Enter sends)"></textarea>
<button id="send">Send</button>
<script>
const API_URL = '';
const history = [];
const log = document.getElementById('log'), box = document.getElementById('box');
function add(role, text){const d=document.createElement('div');d.className=role;d.textContent=role+': '+text;log.appendChild(d);return d;}
async function send(){
  const text = box.value.trim(); if(!text) return; box.value='';
  history.push({role:'user',content:text}); add('user',text);
  const out = add('assistant',''); let reply='';
  const resp = await fetch(API_URL+'/chat/completions',{method:'POST',headers:{'Content-Type':'application/json'},body:JSON.stringify({messages:history})});
  if(!resp.ok){out.textContent='error: '+(await resp.text());history.pop();return;}
  const reader = resp.body.getReader(), dec = new TextDecoder(); let buf='';
  for(;;){const {done,value}=await reader.read(); if(done) break; buf+=dec.decode(value,{stream:true});
    let i; while((i=buf.indexOf('\\n\\n'))>=0){const line=buf.slice(0,i); buf=buf.slice(i+2);
      if(line.startsWith('data: ')){const m=JSON.parse(line.slice(6)); if(m.token){reply+=m.token; out.textContent='assistant: '+reply;}}}}
  history.push({role:'assistant',content:reply});
}
document.getElementById('send').onclick=send;
box.addEventListener('keydown',e=>{if(e.key==='Enter'&&e.ctrlKey)send();});
</script></body></html>"""


class ChatMessage(BaseModel):
    role: str
    content: str


class ChatRequest(BaseModel):
    messages: list[ChatMessage]
    temperature: float | None = None
    max_tokens: int | None = None
    top_k: int | None = None


def _bad(detail: str):
    raise HTTPException(status_code=400, detail=detail)


def validate_chat_request(req: ChatRequest) -> None:
    if not req.messages:
        _bad("At least one message is required")
    if len(req.messages) > MAX_MESSAGES_PER_REQUEST:
        _bad(f"Too many messages. Maximum {MAX_MESSAGES_PER_REQUEST} messages allowed per request")
    total = 0
    for i, m in enumerate(req.messages):
        if not m.content:
            _bad(f"Message {i} has empty content")
        if len(m.content) > MAX_MESSAGE_LENGTH:
            _bad(f"Message {i} is too long. Maximum {MAX_MESSAGE_LENGTH} characters allowed per message")
        if m.role not in ("user", "assistant"):
            _bad(f"Message {i} has invalid role. Must be 'user' or 'assistant'")
        total += len(m.content)
    if total > MAX_TOTAL_CONVERSATION_LENGTH:
        _bad(f"Total conversation is too long. Maximum {MAX_TOTAL_CONVERSATION_LENGTH} characters allowed")
    for name, value, (lo, hi) in (("Temperature", req.temperature, TEMPERATURE_RANGE), ("top_k", req.top_k, TOP_K_RANGE),
                                  ("max_tokens", req.max_tokens, MAX_TOKENS_RANGE)):
        if value is not None and not (lo <= value <= hi):
            _bad(f"{name} must be between {lo} and {hi}")


@dataclass
class Worker:
    gpu_id: int
    device: torch.device
    engine: ChatEngine


class WorkerPool:
    """One engine per GPU (or a single CPU engine); ``acquire`` waits for a free one."""

    def __init__(self, engines: list[ChatEngine]):
        self.workers = [Worker(i, e.device, e) for i, e in enumerate(engines)]
        self.num_gpus = len(self.workers)
        self.available: asyncio.Queue = asyncio.Queue()
        for w in self.workers:
            self.available.put_nowait(w)

    @classmethod
    def load(cls, checkpoint: str, num_gpus: int | None, device_type: str, dtype: str) -> "WorkerPool":
        device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        if device_type != "cuda":
            assert not num_gpus or num_gpus == 1, "only CUDA supports several workers"
            return cls([load_engine(checkpoint, "cpu", "float32")])
        n = num_gpus or torch.cuda.device_count()
        return cls([load_engine(checkpoint, f"cuda:{i}", dtype) for i in range(n)])

    async def acquire(self) -> Worker:
        return await self.available.get()

    async def release(self, w: Worker) -> None:
        await self.available.put(w)


async def _aiter_blocking(gen):
    """Drive a blocking generator from the event loop, one item per worker-thread hop."""
    sentinel = object()
    while (item := await asyncio.to_thread(next, gen, sentinel)) is not sentinel:
        yield item


def create_app(pool: WorkerPool | None = None, *, checkpoint: str | None = None, num_gpus: int | None = 1,
               device_type: str = "", dtype: str = "bfloat16", temperature: float = 0.8, top_k: int = 50,
               max_tokens: int = 512) -> FastAPI:
    @asynccontextmanager
    async def lifespan(app: FastAPI):
        app.state.worker_pool = pool if pool is not None else WorkerPool.load(checkpoint, num_gpus, device_type, dtype)
        yield

    app = FastAPI(lifespan=lifespan)
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"], allow_headers=["*"])

    @app.get("/")
    async def root():
        return HTMLResponse(content=PAGE)

    @app.post("/chat/completions")
    async def chat_completions(request: ChatRequest):
        validate_chat_request(request)
        for m in request.messages:
            logger.info(f"[{m.role.upper()}]: {m.content}")
        wp: WorkerPool = app.state.worker_pool
        worker = await wp.acquire()
        params = SamplingParams(
            n=1,
            max_tokens=request.max_tokens if request.max_tokens is not None else max_tokens,
            temperature=request.temperature if request.temperature is not None else temperature,
            top_k=request.top_k if request.top_k is not None else top_k,
            stop_token_ids=worker.engine.default_stop_ids(),
        )
        messages = [m.model_dump() for m in request.messages]

        async def stream_and_release():
            pieces = []
            try:
                async for piece in _aiter_blocking(worker.engine.stream(messages, params)):
                    pieces.append(piece)
                    yield f"data: {json.dumps({'token': piece, 'gpu': worker.gpu_id}, ensure_ascii=False)}\n\n"
                yield f"data: {json.dumps({'done': True})}\n\n"
            finally:
                logger.info(f"[ASSISTANT] (GPU {worker.gpu_id}): {''.join(pieces)}")
                await wp.release(worker)

        return StreamingResponse(stream_and_release(), media_type="text/event-stream")

    @app.get("/health")
    async def health():
        wp = getattr(app.state, "worker_pool", None)
        return {"status": "ok", "ready": wp is not None and len(wp.workers) > 0, "num_gpus": wp.num_gpus if wp else 0,
                "available_workers": wp.available.qsize() if wp else 0}

    @app.get("/stats")
    async def stats():
        wp: WorkerPool = app.state.worker_pool
        workers = []
        for w in wp.workers:
            entry = {"gpu_id": w.gpu_id, "device": str(w.device)}
            if w.device.type == "cuda":
                entry["memory_allocated_gb"] = torch.cuda.memory_allocated(w.device) / 2**30
            workers.append(entry)
        return {"total_workers": len(wp.workers), "available_workers": wp.available.qsize(),
                "busy_workers": len(wp.workers) - wp.available.qsize(), "workers": workers}

    return app


def main(argv=None):
    p = argparse.ArgumentParser(description="Web chat server")
    p.add_argument("-n", "--num-gpus", type=int, default=1)
    p.add_argument("--checkpoint", type=str, required=True, help="converted HF directory or native .pt checkpoint")
    p.add_argument("-t", "--temperature", type=float, default=0.8)
    p.add_argument("-k", "--top-k", type=int, default=50)
    p.add_argument("-m", "--max-tokens", type=int, default=512)
    p.add_argument("-p", "--port", type=int, default=8000)
    p.add_argument("-d", "--dtype", type=str, default="bfloat16", choices=["float32", "bfloat16"])
    p.add_argument("--device-type", type=str, default="", choices=["", "cuda", "cpu"])
    p.add_argument("--host", type=str, default="0.0.0.0")
    a = p.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s - %(message)s", datefmt="%Y-%m-%d %H:%M:%S")
    import uvicorn

    app = create_app(checkpoint=a.checkpoint, num_gpus=a.num_gpus, device_type=a.device_type, dtype=a.dtype,
                     temperature=a.temperature, top_k=a.top_k, max_tokens=a.max_tokens)
    print(f"Server ready at http://localhost:{a.port}")
    uvicorn.run(app, host=a.host, port=a.port)


if __name__ == "__main__":
    main()
