"""Load-balancing front for the replicas, the role nginx plays in the reference
(utils/generate_compose.py:146-188): listens on one port, forwards every request to one of the
back ends and streams the response through unbuffered.  Policy ``round_robin`` (what the
reference documents, README.md:86) or ``least_conn`` (what its nginx.conf sets,
utils/generate_compose.py:162).

    python -m awq_b200.serving.front --port 8080 --backend http://127.0.0.1:8000 ...
"""
from __future__ import annotations

import argparse
import itertools

HOP_HEADERS = {"connection", "keep-alive", "proxy-authenticate", "proxy-authorization", "te",
               "trailers", "transfer-encoding", "upgrade", "content-length", "host"}


class Balancer:
    """Back-end choice; ``acquire`` / ``release`` bracket one proxied request."""

    def __init__(self, backends: list[str], policy: str = "round_robin") -> None:
        if not backends:
            raise ValueError("at least one back end")
        if policy not in ("round_robin", "least_conn"):
            raise ValueError("policy is 'round_robin' or 'least_conn'")
        self.backends = list(backends)
        self.policy = policy
        self.active = [0] * len(backends)
        self.served = [0] * len(backends)
        self._next = itertools.cycle(range(len(backends)))

    def acquire(self) -> int:
        if self.policy == "round_robin":
            i = next(self._next)
        else:
            # fewest requests in flight; ties go round so an idle pool still spreads
            start = next(self._next)
            order = [(start + j) % len(self.backends) for j in range(len(self.backends))]
            i = min(order, key=lambda b: self.active[b])
        self.active[i] += 1
        self.served[i] += 1
        return i

    def release(self, i: int) -> None:
        self.active[i] -= 1


def make_app(backends: list[str], policy: str = "round_robin"):
    import aiohttp
    from aiohttp import web

    balancer = Balancer(backends, policy)
    state: dict = {}

    async def on_startup(app):
        state["session"] = aiohttp.ClientSession(
            timeout=aiohttp.ClientTimeout(total=None, sock_connect=600, sock_read=600),
            connector=aiohttp.TCPConnector(limit=0), auto_decompress=False)

    async def on_cleanup(app):
        await state["session"].close()

    async def stats(request):
        return web.json_response({"backends": balancer.backends, "served": balancer.served,
                                  "active": balancer.active, "policy": balancer.policy})

    async def forward(request):
        i = balancer.acquire()
        try:
            url = balancer.backends[i].rstrip("/") + request.rel_url.path_qs
            headers = {k: v for k, v in request.headers.items() if k.lower() not in HOP_HEADERS}
            body = await request.read()
            async with state["session"].request(request.method, url, headers=headers,
                                                data=body) as resp:
                out = web.StreamResponse(status=resp.status, headers={
                    k: v for k, v in resp.headers.items() if k.lower() not in HOP_HEADERS})
                await out.prepare(request)
                async for chunk in resp.content.iter_any():
                    await out.write(chunk)
                await out.write_eof()
                return out
        finally:
            balancer.release(i)

    app = web.Application(client_max_size=64 << 20)
    app.on_startup.append(on_startup)
    app.on_cleanup.append(on_cleanup)
    app.router.add_get("/front/stats", stats)
    app.router.add_route("*", "/{tail:.*}", forward)
    app["balancer"] = balancer
    return app


def main() -> None:
    from aiohttp import web
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--backend", action="append", required=True)
    ap.add_argument("--policy", default="round_robin", choices=["round_robin", "least_conn"])
    args = ap.parse_args()
    web.run_app(make_app(args.backend, args.policy), host="127.0.0.1", port=args.port,
                access_log=None, print=None)


if __name__ == "__main__":
    main()
