"""Request accounting in SQLite: one row per finished request (tokens in/out, cache hits, latency, finish reason),
daily roll-ups for the usage endpoint, optional 24-hour prompt log with redaction.
Reference: cuteafd-usage/src/{store,query,daily}.rs, README.md:222-224."""
from __future__ import annotations

import re
import sqlite3
import threading
import time

SECRET = re.compile(r"(sk-[A-Za-z0-9]{8,}|Bearer\s+[A-Za-z0-9._-]{8,}|[A-Za-z0-9._%+-]+@[A-Za-z0-9.-]+\.[a-z]{2,})")


class UsageStore:
    def __init__(self, path: str = ":memory:", keep_log_hours: float = 24.0, log_prompts: bool = False):
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.lock = threading.Lock()
        self.keep_s, self.log_prompts = keep_log_hours * 3600, log_prompts
        self.db.executescript("""
            create table if not exists requests(id text primary key, t real, model text, api_key text, prompt_tokens int,
                completion_tokens int, cache_hit_tokens int, ttft_ms real, total_ms real, finish text);
            create table if not exists prompt_log(id text primary key, t real, text text);""")

    def record(self, rid, model, api_key, prompt_tokens, completion_tokens, cache_hit_tokens, ttft_ms, total_ms, finish, prompt_text=None, now=None):
        now = now or time.time()
        with self.lock:
            self.db.execute("insert or replace into requests values(?,?,?,?,?,?,?,?,?,?)",
                            (rid, now, model, api_key, prompt_tokens, completion_tokens, cache_hit_tokens, ttft_ms, total_ms, finish))
            if self.log_prompts and prompt_text is not None:
                self.db.execute("insert or replace into prompt_log values(?,?,?)", (rid, now, SECRET.sub("[redacted]", prompt_text)))
            self.db.execute("delete from prompt_log where t < ?", (now - self.keep_s,))
            self.db.commit()

    def daily(self) -> list[dict]:
        with self.lock:
            cur = self.db.execute("""select date(t, 'unixepoch'), count(*), sum(prompt_tokens), sum(completion_tokens), sum(cache_hit_tokens),
                                     avg(ttft_ms) from requests group by 1 order by 1""")
            return [{"day": d, "requests": n, "prompt_tokens": p, "completion_tokens": c, "cache_hit_tokens": h, "avg_ttft_ms": t}
                    for d, n, p, c, h, t in cur.fetchall()]

    def by_key(self) -> list[dict]:
        with self.lock:
            cur = self.db.execute("select api_key, count(*), sum(prompt_tokens + completion_tokens) from requests group by 1")
            return [{"api_key": k, "requests": n, "tokens": t} for k, n, t in cur.fetchall()]

    # ------------------------------------------------------------------ maintenance (the `usage` command)
    RANGES = {"1h": 3600.0, "6h": 6 * 3600.0, "24h": 86400.0, "7d": 7 * 86400.0}

    def clear(self):
        """Both tiers: request metadata and the prompt log."""
        with self.lock:
            self.db.executescript("delete from requests; delete from prompt_log;")
            self.db.commit()

    def clear_log(self):
        """Only the prompt log (payloads); metadata stays."""
        with self.lock:
            self.db.execute("delete from prompt_log")
            self.db.commit()

    def export_csv(self, out, range_: str = "7d", now=None) -> int:
        """Request metadata of the range ending now as CSV (never payloads).  Returns rows written."""
        import csv
        now = now or time.time()
        with self.lock:
            rows = self.db.execute("select id, t, model, api_key, prompt_tokens, completion_tokens, cache_hit_tokens, ttft_ms, total_ms, finish "
                                   "from requests where t >= ? order by t", (now - self.RANGES[range_],)).fetchall()
        w = csv.writer(out)
        w.writerow(["id", "time", "model", "api_key", "prompt_tokens", "completion_tokens", "cache_hit_tokens", "ttft_ms", "total_ms", "finish"])
        w.writerows(rows)
        return len(rows)

    def totals(self) -> dict:
        with self.lock:
            n, p, c, h = self.db.execute("select count(*), coalesce(sum(prompt_tokens),0), coalesce(sum(completion_tokens),0), "
                                         "coalesce(sum(cache_hit_tokens),0) from requests").fetchone()
        return {"requests": n, "prompt_tokens": p, "completion_tokens": c, "cache_hit_tokens": h}


def synthetic_history(store: UsageStore, days: int = 7, per_day: int = 40, seed: int = 0, now=None):
    """Fills a store with a plausible request history (the usage page can be developed without a GPU or a model)."""
    import random
    rng, now = random.Random(seed), now or time.time()
    for d in range(days):
        for i in range(per_day):
            t = now - d * 86400 - rng.random() * 86000
            p, c = rng.randrange(50, 30000), rng.randrange(1, 2000)
            store.record(f"demo-{d}-{i}", "demo-model", rng.choice(["key-a", "key-b", "key-c"]), p, c, rng.choice([0, 0, (p // 64) * 64 // 2]),
                         rng.uniform(20, 3000), rng.uniform(100, 60000), rng.choice(["stop", "length", "tool_calls"]), now=t)
