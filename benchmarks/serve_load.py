"""Load test of the OpenAI-compatible server: N concurrent streaming requests of random prompt ids.

    python benchmarks/serve_load.py --model random:llama-3-70b --gpus 8 --requests 64 --prompt 1024 --output 256 \
        --shared-prefix 512 --shared-frac 0.5 --rows 64 --max-seq 2048

Starts the server (one process per GPU under ``torch.distributed.run`` when ``--gpus > 1``), waits for ``/health``,
runs the workload ``--waves`` times (the first wave warms up the captured step shapes) and prints one JSON line for
the last wave: aggregate output tok/s, prompt tok/s, TTFT and inter-token latency percentiles as seen by the client,
and the server's own prefix-cache counters.  All times are host wall-clock around HTTP calls: this is the
end-to-end serving number, not a kernel time.
"""
import argparse
import http.client
import json
import os
import random
import signal
import subprocess
import sys
import threading
import time


def pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else 0.0


def get(port, path, timeout=5):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=timeout)
    c.request("GET", path)
    r = c.getresponse()
    body = r.read()
    c.close()
    return r.status, body


def one_request(port, prompt, n_out, rec):
    body = json.dumps({"prompt": prompt, "max_tokens": n_out, "temperature": 0, "ignore_eos": True, "stream": True})
    t0 = time.perf_counter()
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=600)
    c.request("POST", "/v1/completions", body, {"Content-Type": "application/json"})
    r = c.getresponse()
    rec["status"] = r.status
    stamps = []
    if r.status == 200:
        while True:
            line = r.readline()
            if not line:
                break
            if line.startswith(b"data: "):
                if line.startswith(b"data: [DONE]"):
                    break
                stamps.append(time.perf_counter())
    c.close()
    rec["t0"], rec["stamps"] = t0, stamps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:llama-3-70b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--output", type=int, default=256)
    ap.add_argument("--shared-prefix", type=int, default=512)
    ap.add_argument("--shared-frac", type=float, default=0.5)
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--max-seq", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--port", type=int, default=8123)
    ap.add_argument("--waves", type=int, default=2)
    ap.add_argument("--startup-timeout", type=float, default=420)
    ap.add_argument("--log", default="serve_load_server.log")
    a = ap.parse_args()

    serve = ["-m", "poot_b200.serve", a.model, f"127.0.0.1:{a.port}", "--rows", str(a.rows), "--max-seq", str(a.max_seq),
             "--prefill-chunk", str(a.prefill_chunk), "--max-pending-requests", str(max(256, 2 * a.requests))]
    if a.gpus > 1:
        serve += ["--placement", "tensor:" + ",".join(map(str, range(a.gpus)))]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533"] + serve
    else:
        cmd = [sys.executable] + serve
    os.makedirs(os.path.dirname(a.log) or ".", exist_ok=True)
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    with open(a.log, "w") as logf:
        proc = subprocess.Popen(cmd, stdout=logf, stderr=subprocess.STDOUT, start_new_session=True, env=env)
    result = {"error": None}
    try:
        t_start = time.time()
        while True:
            if proc.poll() is not None:
                raise RuntimeError(f"server exited with {proc.returncode} during startup (see {a.log})")
            try:
                if get(a.port, "/health")[0] == 200:
                    break
            except OSError:
                pass
            if time.time() - t_start > a.startup_timeout:
                raise RuntimeError("server did not become healthy in time")
            time.sleep(1.0)
        startup_s = time.time() - t_start
        rng = random.Random(0)
        for wave in range(a.waves):
            shared = [rng.randrange(3, a.vocab) for _ in range(a.shared_prefix)]
            prompts = []
            for i in range(a.requests):
                if i < int(a.requests * a.shared_frac):
                    p = shared + [rng.randrange(3, a.vocab) for _ in range(a.prompt - a.shared_prefix)]
                else:
                    p = [rng.randrange(3, a.vocab) for _ in range(a.prompt)]
                prompts.append(p)
            rng.shuffle(prompts)
            recs = [dict() for _ in prompts]
            m0 = json.loads(get(a.port, "/metrics")[1])["counters"]
            t0 = time.perf_counter()
            ts = [threading.Thread(target=one_request, args=(a.port, p, a.output, r)) for p, r in zip(prompts, recs)]
            [t.start() for t in ts]
            [t.join() for t in ts]
            wall = time.perf_counter() - t0
            m1 = json.loads(get(a.port, "/metrics")[1])["counters"]
            ok = [r for r in recs if r.get("status") == 200 and r.get("stamps")]
            ttft = [(r["stamps"][0] - r["t0"]) * 1e3 for r in ok]
            itl = [(b - x) * 1e3 for r in ok for x, b in zip(r["stamps"], r["stamps"][1:])]
            out_tokens = m1["poot_completion_tokens_total"] - m0["poot_completion_tokens_total"]
            result = {
                "metric": "server output tok/s (aggregate, client wall clock)", "value": out_tokens / wall, "unit": "tok/s",
                "n_gpus": a.gpus, "wave": wave, "requests": a.requests, "completed": len(ok), "wall_s": wall,
                "prompt_tok_s": a.requests * a.prompt / wall, "ttft_ms": {"p50": pct(ttft, 0.5), "p95": pct(ttft, 0.95)},
                "itl_ms": {"p50": pct(itl, 0.5), "p95": pct(itl, 0.95)},
                "prefix_cache_hit_tokens": m1["poot_prefix_cache_hit_tokens_total"] - m0["poot_prefix_cache_hit_tokens_total"],
                "engine_steps": m1["poot_engine_steps_total"] - m0["poot_engine_steps_total"], "startup_s": startup_s,
                "config": {"model": a.model, "prompt": a.prompt, "output": a.output, "shared_prefix": a.shared_prefix,
                           "shared_frac": a.shared_frac, "rows": a.rows, "max_seq": a.max_seq, "kv": "paged block 16, prefix cache on",
                           "parallelism": f"tp{a.gpus}", "data": "synthetic token ids, random-init weights"},
            }
            print(json.dumps(result), flush=True)
    except Exception as e:      # report and still shut the server down
        result = {"error": str(e)}
        print(json.dumps(result), flush=True)
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)     # the server's own process group only
            proc.wait(timeout=60)
        except Exception:
            try:
                os.killpg(proc.pid, signal.SIGKILL)
            except Exception:
                pass
    return 0 if not result.get("error") else 1


if __name__ == "__main__":
    sys.exit(main())
