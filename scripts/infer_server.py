"""Minimal OpenAI-compatible chat server on the framework's own Qwen3 model (one GPU, or CPU).

    python scripts/infer_server.py --model out_hf --flavor 1.7B --tokenizer assets/hf/Qwen3-1.7B --port 8000
    curl localhost:8000/v1/chat/completions -d '{"messages": [{"role": "user", "content": "hi"}]}'

``--model`` is a folder of Hugging Face safetensors (e.g. the output of checkpoint_conversion/convert_to_hf.py, or the
released weights); they are mapped to native names by the model's state-dict adapter.  Decoding recomputes the prefix
every step (no KV cache): meant for checking a freshly fine-tuned checkpoint, not for serving load.

(reference: scripts/infer_server.py:19-83)
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import sys
import time
from http.server import BaseHTTPRequestHandler, HTTPServer

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load(model_path: str, module: str, flavor: str, tokenizer_path: str | None, device: str):
    from safetensors.torch import load_file

    from titan_b200.data.tokenizer import build_tokenizer
    from titan_b200.protocols.model_spec import get_model_spec

    spec = get_model_spec(module, flavor)
    cfg = spec.model
    with torch.device("meta"):
        model = cfg.build()
    model.to_empty(device=device)
    model.init_states(buffer_device=torch.device(device))
    hf = {}
    for f in sorted(glob.glob(os.path.join(model_path, "*.safetensors"))):
        hf.update(load_file(f))
    if not hf:
        raise FileNotFoundError(f"no *.safetensors under {model_path!r}")
    native = spec.state_dict_adapter(cfg, model_path).from_hf(hf)
    missing, unexpected = model.load_state_dict(native, strict=False)
    missing = [k for k in missing if "expert_bias" not in k and "tokens_per_expert" not in k]
    if missing or unexpected:
        raise RuntimeError(f"checkpoint / model mismatch: missing {missing[:5]}, unexpected {list(unexpected)[:5]}")
    model.to(torch.bfloat16 if device != "cpu" else torch.float32).eval()
    return build_tokenizer(tokenizer_path or model_path), model


@torch.inference_mode()
def generate(model, tok, ids: list[int], max_new_tokens: int, temperature: float, device: str) -> list[int]:
    out = []
    x = torch.tensor([ids], device=device)
    limit = model.config.max_seq_len
    stop = {tok.eos_id} | set(tok.encode("<|im_end|>", add_bos=False, add_eos=False)[:1])
    for _ in range(max_new_tokens):
        if x.shape[1] >= limit:
            break
        logits = model(x)[0, -1].float()
        if temperature > 0:
            nxt = int(torch.multinomial(torch.softmax(logits / temperature, -1), 1))
        else:
            nxt = int(logits.argmax())
        if nxt in stop:
            break
        out.append(nxt)
        x = torch.cat([x, torch.tensor([[nxt]], device=device)], dim=1)
    return out


class Handler(BaseHTTPRequestHandler):
    def do_POST(self):
        req = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
        srv = self.server
        text = srv.tokenizer.apply_chat_template(req.get("messages", []), tokenize=False, add_generation_prompt=True)
        ids = srv.tokenizer.encode(text, add_bos=True, add_eos=False)
        t0 = time.time()
        new = generate(srv.model, srv.tokenizer, ids, int(req.get("max_tokens", 1024)),
                       float(req.get("temperature", 0.6)), srv.device)
        reply = srv.tokenizer.decode(new)
        self._json({"id": f"chatcmpl-{int(t0)}", "object": "chat.completion", "created": int(t0),
                    "model": req.get("model", srv.model_name),
                    "choices": [{"index": 0, "finish_reason": "stop",
                                 "message": {"role": "assistant", "content": reply}}],
                    "usage": {"prompt_tokens": len(ids), "completion_tokens": len(new),
                              "total_tokens": len(ids) + len(new)}})
        print(f"[{time.time() - t0:.1f}s] {reply[:80]}...")

    def do_GET(self):
        if self.path == "/health":
            self._json({"status": "ok"})
        else:
            self._json({"error": "not found"}, 404)

    def _json(self, data, status=200):
        body = json.dumps(data).encode()
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.end_headers()
        self.wfile.write(body)


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="./assets/hf/Qwen3-1.7B")
    p.add_argument("--module", default="qwen3")
    p.add_argument("--flavor", default="1.7B")
    p.add_argument("--tokenizer", default=None, help="tokenizer asset folder (default: the model folder)")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    args = p.parse_args()
    server = HTTPServer((args.host, args.port), Handler)
    server.device, server.model_name = args.device, f"{args.module}-{args.flavor}"
    server.tokenizer, server.model = load(args.model, args.module, args.flavor, args.tokenizer, args.device)
    server.serve_forever()
