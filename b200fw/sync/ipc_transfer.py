"""vLLM-server compatibility layer: HTTP control client, CUDA-IPC handle transfer, and the weight update
manager with rollback (src/transfer/ipc_transfer.py:53-667).

Not on this framework's product path (rollouts run in the native engine and weights move by peer
write), but kept so that a vLLM server can still be driven: the same endpoints, the same retry taxonomy
(programming errors are never retried, a CUDA out-of-memory answer is retried once, everything else
with linear back-off), chunked handle payloads keyed by GPU UUID, and ``push_weights`` always tries to
wake the server up again when something fails.
"""
from __future__ import annotations

import asyncio
import base64
import hashlib
import pickle
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch

from ..obs.logging import get_logger
from .nccl_transfer import TransferStats
from ..compat import kwarg_aliases

logger = get_logger("sync.ipc")


class NonRetriableError(Exception):
    pass


# The retry taxonomy under the reference's names (src/transfer/ipc_transfer.py:53-65): network-side failures are worth
# another attempt, malformed data is not.  ``classify_error`` is what the client consults.
RETRIABLE_EXCEPTIONS = (TimeoutError, ConnectionError, OSError)
NON_RETRIABLE_EXCEPTIONS = (ValueError, KeyError, TypeError, NonRetriableError)


def classify_error(e: BaseException) -> str:
    """'fatal' (never retry), 'oom' (retry once), or 'retry'."""
    if isinstance(e, NON_RETRIABLE_EXCEPTIONS):
        return "fatal"
    if "out of memory" in str(e).lower():
        return "oom"
    return "retry"


class VLLMClient:
    def __init__(self, base_url: str = "http://localhost:8000", timeout: float = 60.0, max_retries: int = 3,
                 backoff_s: float = 1.0, client=None, retry_delay: Optional[float] = None):
        self.base_url = base_url.rstrip("/")
        backoff_s = retry_delay if retry_delay is not None else backoff_s      # `retry_delay`: the reference's name
        self.timeout, self.max_retries, self.backoff_s = timeout, max_retries, backoff_s
        self._client = client
        self.calls: List[str] = []

    async def _get_client(self):
        if self._client is None:
            import httpx
            self._client = httpx.AsyncClient(base_url=self.base_url, timeout=httpx.Timeout(self.timeout))
        return self._client

    async def _request(self, method: str, path: str, **kw) -> Any:
        """One request with the retry policy; ``path`` is relative to the client's base URL.  ``None``-valued
        keyword arguments are dropped, so a call without parameters reaches the HTTP client as ``get("/health")``."""
        client = await self._get_client()
        kw = {k: v for k, v in kw.items() if v is not None}
        attempt, oom_retried = 0, False
        while True:
            try:
                self.calls.append(f"{method} {path}")
                resp = await getattr(client, method.lower())(path, **kw)
                if hasattr(resp, "raise_for_status"):
                    resp.raise_for_status()
                return resp
            except Exception as e:  # noqa: BLE001
                kind = classify_error(e)
                attempt += 1
                if kind == "fatal":
                    raise
                if kind == "oom":
                    if oom_retried:
                        raise
                    oom_retried = True
                elif attempt > self.max_retries:
                    raise
                await asyncio.sleep(self.backoff_s * attempt)

    # ---- control endpoints of the vLLM server (src/transfer/ipc_transfer.py:215-287): every call returns True and
    # raises when the server refuses after the retries ------------------------------------------------------
    async def health(self) -> bool:
        try:
            resp = await self._request("GET", "/health")
            return getattr(resp, "status_code", 200) == 200
        except Exception:  # noqa: BLE001
            return False

    async def health_check(self) -> bool:
        return await self.health()

    async def reset_prefix_cache(self) -> bool:
        await self._request("POST", "/reset_prefix_cache",
                            params={"reset_running_requests": False, "reset_external": False})
        return True

    async def sleep(self, level: int = 1) -> bool:
        """Level 0 pauses scheduling, 1 offloads weights and drops the KV cache, 2 frees all device memory.  The
        prefix cache is reset first (a failure there is not fatal)."""
        try:
            await self.reset_prefix_cache()
        except Exception as e:  # noqa: BLE001
            logger.warning("reset_prefix_cache failed (non-fatal): %s", e)
        await self._request("POST", "/sleep", params={"level": level})
        return True

    async def wake_up(self, tags=None) -> bool:
        """``tags``: a list such as ``["weights", "kv_cache"]`` (sent as repeated query parameters) or one tag."""
        if isinstance(tags, str):
            tags = [tags]
        await self._request("POST", "/wake_up", params={"tags": list(tags)} if tags else None)
        return True

    async def completions(self, prompt: str, n: int = 1, max_tokens: int = 512, temperature: float = 0.7,
                          top_p: float = 0.95, model: Optional[str] = None) -> List[str]:
        """``n`` sampled continuations of ``prompt`` through the server's OpenAI-style ``/v1/completions`` endpoint
        (the rollout call of the reference's vLLM backend: src/orchestrator/colocate_orchestrator.py:1406-1433)."""
        body = {"prompt": prompt, "n": n, "max_tokens": max_tokens, "temperature": temperature, "top_p": top_p}
        if model:
            body["model"] = model
        resp = await self._request("POST", "/v1/completions", json=body)
        return [c["text"] for c in resp.json()["choices"]]

    async def init_weight_transfer(self, init_info: Optional[Dict] = None) -> bool:
        await self._request("POST", "/init_weight_transfer_engine", json={"init_info": init_info or {}})
        return True

    async def start_weight_update(self, is_checkpoint_format=True) -> bool:
        if isinstance(is_checkpoint_format, dict):           # older call style: a ready-made body
            body = is_checkpoint_format
        else:
            body = {"is_checkpoint_format": bool(is_checkpoint_format)}
        await self._request("POST", "/start_weight_update", json=body)
        return True

    async def update_weights(self, update_info: Dict, weight_version: Optional[str] = None) -> bool:
        body: Dict[str, Any] = {"update_info": update_info}
        if weight_version is not None:
            body["weight_version"] = weight_version
        await self._request("POST", "/update_weights", json=body)
        return True

    async def finish_weight_update(self) -> bool:
        await self._request("POST", "/finish_weight_update", json={})
        return True

    async def close(self):
        if self._client is not None and hasattr(self._client, "aclose"):
            await self._client.aclose()
        self._client = None


def _gpu_uuid(device_index: int = 0) -> str:
    try:
        return str(torch.cuda.get_device_properties(device_index).uuid)
    except Exception:  # noqa: BLE001
        return f"cpu-{device_index}"


@dataclass
class IPCHandle:
    """One exported tensor (src/transfer/ipc_transfer.py:68-75); ``build_ipc_handles`` produces the same records
    as plain dicts with these keys."""
    name: str
    handle: object
    shape: tuple
    dtype: torch.dtype
    device_id: int = 0


class IPCWeightTransfer:
    def __init__(self, client: Optional[VLLMClient] = None, chunk_size: int = 16, device_index: int = 0,
                 vllm_client: Optional[VLLMClient] = None):
        client = client if client is not None else vllm_client                  # `vllm_client`: the reference's name
        assert client is not None, "IPCWeightTransfer needs a VLLMClient"
        self.client, self.chunk_size, self.device_index = client, chunk_size, device_index
        self.stats = TransferStats()
        self._keepalive: List[torch.Tensor] = []     # exported tensors must outlive the receiver's import

    @kwarg_aliases(state_dict="state")
    def build_ipc_handles(self, state: Dict[str, torch.Tensor]) -> List[Dict]:
        handles = []
        self._keepalive = []
        for name, t in state.items():
            t = t.detach().contiguous()
            self._keepalive.append(t)
            if t.is_cuda:
                from torch.multiprocessing.reductions import reduce_tensor
                fn, args = reduce_tensor(t)
                handle = (fn.__name__, args)
            else:
                handle = ("cpu_tensor", t)        # CPU fallback keeps the protocol testable
            handles.append({"name": name, "shape": tuple(t.shape), "dtype": str(t.dtype), "handle": handle})
        return handles

    def _chunk_handles(self, handles: List[Dict]) -> List[List[Dict]]:
        return [handles[i:i + self.chunk_size] for i in range(0, len(handles), self.chunk_size)]

    def _build_http_payload(self, chunk: List[Dict]) -> Dict:
        blob = base64.b64encode(pickle.dumps([h["handle"] for h in chunk])).decode()
        return {"names": [h["name"] for h in chunk], "shapes": [list(h["shape"]) for h in chunk],
                "dtypes": [h["dtype"] for h in chunk], "ipc_handles": {_gpu_uuid(self.device_index): blob}}

    def push_weights_sync(self, state_dict: Dict[str, torch.Tensor], sleep_level: int = 0) -> bool:
        """Blocking wrapper around :meth:`push_weights` (a worker thread when an event loop is already running);
        ``sleep_level > 0`` puts the server to sleep first.  Returns whether the push went through."""
        import concurrent.futures

        def run():
            return asyncio.run(self.push_weights(state_dict, sleep_first=sleep_level > 0))
        try:
            try:
                asyncio.get_running_loop()
            except RuntimeError:
                run()
            else:
                with concurrent.futures.ThreadPoolExecutor(1) as pool:
                    pool.submit(run).result()
            return True
        except Exception as e:  # noqa: BLE001 - reported as the return value, as the reference does
            logger.error("push_weights failed: %s", e)
            return False

    def verify_consistency(self, local_dict: Dict[str, torch.Tensor], remote_checksum: Optional[str] = None) -> bool:
        """md5 over the full tensors in name order against the receiver's checksum (``True`` when none is given)."""
        return remote_checksum is None or self.checksum(local_dict) == remote_checksum

    def release_refs(self):
        """Drop the references that keep exported tensors alive (only after the receiver has imported them)."""
        self._keepalive.clear()

    @staticmethod
    def checksum(state: Dict[str, torch.Tensor]) -> str:
        m = hashlib.md5()
        for k in sorted(state):
            m.update(k.encode())
            m.update(state[k].detach().to(torch.float32).cpu().contiguous().numpy().tobytes())
        return m.hexdigest()

    @kwarg_aliases(state_dict="state", sleep_level="sleep_first")
    async def push_weights(self, state: Dict[str, torch.Tensor], sleep_first: bool = True) -> TransferStats:
        t0 = time.perf_counter()
        nbytes = sum(v.numel() * v.element_size() for v in state.values())
        try:
            if sleep_first:
                await self.client.sleep()
            handles = self.build_ipc_handles(state)
            await self.client.init_weight_transfer()
            await self.client.start_weight_update(True)
            for chunk in self._chunk_handles(handles):
                await self.client.update_weights(self._build_http_payload(chunk))
            await self.client.finish_weight_update()
            await self.client.wake_up()
            self.stats.record(nbytes, time.perf_counter() - t0, ok=True)
        except Exception:
            self.stats.record(nbytes, time.perf_counter() - t0, ok=False)
            try:
                await self.client.wake_up()      # never leave the server asleep
            except Exception as e2:  # noqa: BLE001
                logger.warning("wake_up after a failed push also failed: %s", e2)
            raise
        return self.stats


class WeightUpdateManager:
    """Apply a state dict to a model; on any failure restore the previous tensors
    (src/transfer/ipc_transfer.py:566-667)."""

    def __init__(self, model: torch.nn.Module, validate: Optional[Callable[[torch.nn.Module], bool]] = None):
        self.model, self.validate = model, validate
        self.version = 0
        self.rollbacks = 0

    @torch.no_grad()
    def update_weights(self, state: Optional[Dict[str, torch.Tensor]] = None, *,
                       new_state_dict: Optional[Dict[str, torch.Tensor]] = None) -> bool:
        state = state if state is not None else new_state_dict      # ``new_state_dict``: the reference's keyword
        params = dict(self.model.named_parameters())
        backup = {k: params[k].detach().clone() for k in state if k in params}
        try:
            for k, v in state.items():
                if k not in params:
                    continue
                if tuple(params[k].shape) != tuple(v.shape):
                    raise ValueError(f"shape mismatch for {k}: {tuple(v.shape)} vs {tuple(params[k].shape)}")
                if not torch.isfinite(v).all():
                    raise ValueError(f"non-finite values in {k}")
                params[k].copy_(v.to(params[k].dtype))
            if self.validate is not None and not self.validate(self.model):
                raise RuntimeError("post-update validation failed")
            self.version += 1
            return True
        except Exception as e:  # noqa: BLE001
            for k, v in backup.items():
                params[k].copy_(v)
            self.rollbacks += 1
            logger.warning("weight update rolled back: %s", e)
            return False

    # the reference's property names (src/transfer/ipc_transfer.py:659-667)
    @property
    def current_version(self) -> int:
        return self.version

    @property
    def rollback_count(self) -> int:
        return self.rollbacks

