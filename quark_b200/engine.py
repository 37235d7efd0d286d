"""``Engine``: the session API of the reference (``quark.Engine``), minus the VAE.

Mirrors ``src/quark/engine/cuda.py:38-51`` / ``:169-266`` and the factory in
``src/quark/engine/base.py:155-165``: ``Engine(cfg, quant=...)``, ``append_frame``, ``gen_frame``,
``reset``.  The reference wraps the DiT between a torch VAE encoder and decoder; the VAE is outside
the hot path, so here ``append_frame`` takes a latent ``[1, C, 2H, 2W]`` and ``gen_frame`` returns
the generated latent (documented deviation).  Each ``gen_frame`` copies the noise latent from
pinned host memory to the device, replays the captured 5-NFE CUDA graph, and copies the
result back: those copies are the only host <-> device traffic per frame.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from .models.waypoint_15 import GenerateFrame, QuantConfig, Waypoint15, Waypoint15Config, make_params
from .runtime import stream as _stream
from .runtime.tensor import QuarkTensor


class _Pinned:
    """A pinned host buffer viewed as a numpy array."""

    def __init__(self, nbytes: int, dtype):
        p = C.c_void_p()
        _lib.check(_lib.load().qb_host_alloc(C.byref(p), nbytes))
        self.ptr = int(p.value)
        self.array = np.frombuffer((C.c_uint8 * nbytes).from_address(self.ptr), dtype=dtype)

    def __del__(self):
        try:
            _lib.load().qb_host_free(C.c_void_p(self.ptr))
        except Exception:
            pass


@dataclass
class CtrlInput:
    """Controller input for one frame (``src/quark/models/waypoint_15.py:38-43``)."""

    button: set = field(default_factory=set)
    mouse: tuple = (0.0, 0.0)
    scroll_wheel: int = 0


class Engine:
    def __init__(self, model_uri=None, *, cfg: Waypoint15Config | None = None, quant="fp8", load_weights=True, seed: int = 0,
                 params: dict | None = None, device: int = 0, use_graph: bool = True, comm=None, device_noise: bool = False,
                 watchdog_s: float | None = None):  # fmt: skip
        if isinstance(model_uri, Waypoint15Config):
            cfg, model_uri = model_uri, None
        if model_uri is not None:
            # a local directory with config.yaml and model.safetensors (src/quark/engine/cuda.py:77, :105-108);
            # only the transformer is read: the autoencoder and the prompt encoder sit outside this package
            from .models.checkpoint import load_checkpoint

            if cfg is None:
                cfg = Waypoint15Config.from_yaml(model_uri)
            if load_weights and params is None:
                params = load_checkpoint(model_uri, cfg)
        _lib.require_device(device)
        _lib.check(_lib.load().qb_set_device(device))
        if isinstance(quant, str):
            quant = QuantConfig.all_fp8() if quant == "fp8" else QuantConfig.all_bf16() if quant == "bf16" else None
            if quant is None:
                raise ValueError("Engine: quant must be 'fp8', 'bf16' or a QuantConfig")
        base = cfg or Waypoint15Config()
        self.cfg = cfg = Waypoint15Config(**{**base.__dict__, "quant": quant})
        self.model = Waypoint15(cfg, comm)
        if load_weights:
            self.model.load_params(params if params is not None else make_params(cfg, seed))
            self.model.prepare()
        self.gen = GenerateFrame(self.model)
        self._use_graph = use_graph
        # A sharded session (comm.world > 1) waits for its peers inside every frame.  With `watchdog_s` set, a frame that
        # takes longer aborts the communicator from a timer thread, so that a rank whose peer died returns with an error
        # instead of waiting inside a collective (runtime.nccl.Watchdog).  The reference is single-GPU: no counterpart.
        self._watchdog = None
        if watchdog_s is not None and comm is not None and getattr(comm, "world", 1) > 1:
            from .runtime.nccl import Watchdog

            self._watchdog = Watchdog(comm, watchdog_s)
        self._frame = 0
        n = cfg.latent_numel
        self._noise_host = _Pinned(n * 2, np.uint16)
        self._out_host = _Pinned(n * 2, np.uint16)
        self._noise_dev = QuarkTensor.empty(1, n, dtype="bf16")
        self._append_dev = QuarkTensor.empty(1, n, dtype="bf16")
        self._rng = np.random.default_rng([seed, 7])
        # device_noise: the frame's starting noise is drawn on the device (qf.randn keyed by the frame counter)
        # instead of on the host, so a frame needs no host-to-device copy (src/quark/functional/randn.py:1-17)
        self._device_noise = bool(device_noise)
        self._noise_seeds = (0xDEADBEEF, (0xBADC0FFE + int(seed)) & 0xFFFFFFFF)
        self.h2d_bytes_per_frame = n * 2
        self.d2h_bytes_per_frame = n * 2
        # persistent controller row (device) and its pinned staging copy; refilled per frame, so the captured
        # graph always reads the same address (src/quark/engine/cuda.py:115-116, models/_waypoint_15_io.py:225-322)
        self._ctrl_dev = self._ctrl_host = None
        if cfg.ctrl_conditioning:
            w = cfg.ctrl_input_width
            self._ctrl_dev = QuarkTensor.zeros(1, w, dtype="bf16")
            self._ctrl_host = _Pinned(w * 2, np.uint16)
            self.h2d_bytes_per_frame += w * 2

    # ---- helpers
    def _latent_shape(self):
        c = self.cfg
        return (1, c.channels, c.height * c.patch[0], c.width * c.patch[1])

    def _to_bf16(self, latent) -> np.ndarray:
        a = np.asarray(latent)
        if a.dtype == np.uint16:
            out = a
        else:
            out = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)
        if out.size != self.cfg.latent_numel:
            raise ValueError(f"Engine: latent has {out.size} elements, expected {self._latent_shape()}")
        return out.reshape(-1)

    def _encode_ctrl(self, ctrl):
        """Packs ``[mouse x, mouse y, one flag per pressed button, scroll wheel]`` (bf16, zero padded) and copies it
        to the persistent device row; None when the model has no controller path.  ``ctrl=None`` is the idle
        controller (all zeros), as upstream."""
        if self._ctrl_dev is None:
            if ctrl is not None:
                raise ValueError("Engine: ctrl given but the model was built with ctrl_conditioning=False")
            return None
        ctrl = ctrl or CtrlInput()
        nb = self.cfg.n_buttons
        row = np.zeros(self.cfg.ctrl_input_width, np.float32)
        row[0], row[1] = float(ctrl.mouse[0]), float(ctrl.mouse[1])
        for b in ctrl.button:
            if 0 <= b < nb:
                row[2 + b] = 1.0
        row[2 + nb] = float(ctrl.scroll_wheel)
        self._ctrl_host.array[:] = (row.view(np.uint32) >> np.uint32(16)).astype(np.uint16)
        self._h2d(self._ctrl_dev, self._ctrl_host.ptr, row.size * 2)
        return self._ctrl_dev

    def _h2d(self, dev: QuarkTensor, host_ptr: int, nbytes: int):
        _lib.check(_lib.load().qb_memcpy_async(C.c_void_p(dev.data_ptr()), C.c_void_p(host_ptr), nbytes, 0, C.c_void_p(_stream.active_stream())))

    def _d2h(self, host_ptr: int, dev: QuarkTensor, nbytes: int):
        _lib.check(_lib.load().qb_memcpy_async(C.c_void_p(host_ptr), C.c_void_p(dev.data_ptr()), nbytes, 1, C.c_void_p(_stream.active_stream())))

    @property
    def launches_per_frame(self) -> int:
        """Kernels in the captured frame graph (0 before the first ``gen_frame``)."""
        return int(self.gen.launches_per_frame)

    def close(self) -> None:
        """Drops the captured frame graph (a communicator whose collectives it holds cannot be destroyed
        before); the engine runs eagerly afterwards unless a new graph is captured."""
        self.gen._graph = None
        self._use_graph = False
        import gc

        gc.collect()
        _stream.synchronize()

    # ---- session API
    def reset(self) -> None:
        self.gen.reset()
        self._frame = 0

    def set_frame_t(self, value: int) -> None:
        self.gen.set_frame_t(value)
        self._frame = int(value)

    def snapshot(self) -> dict:
        """The session's state as host arrays: every layer's caches and segment table, the frame counter and
        the host noise generator.  ``restore`` brings a session (of the same configuration) back to it, so a
        continuation can be replayed or branched.  The reference has no counterpart (its engine can only
        ``reset``, ``src/quark/engine/base.py:187-195``)."""
        _stream.synchronize()
        layers = []
        for blk in self.model.blocks:
            kc = blk.kv_cache
            layers.append({k: getattr(kc, k).to_numpy().copy() for k in ("K_cache", "Vt_cache", "segments", "n_segments")})
        return {"layers": layers, "frame_t": int(self.gen.frame_t.to_numpy()[0]), "frame": self._frame,
                "rng": self._rng.bit_generator.state, "geometry": (self.cfg.n_layers, self.cfg.tpf, str(self.cfg.quant.kv_cache))}  # fmt: skip

    def restore(self, snap: dict) -> None:
        if snap.get("geometry") != (self.cfg.n_layers, self.cfg.tpf, str(self.cfg.quant.kv_cache)):
            raise ValueError(f"Engine.restore: snapshot of {snap.get('geometry')} does not fit this engine")
        _stream.synchronize()
        for blk, saved in zip(self.model.blocks, snap["layers"]):
            for k, host in saved.items():
                getattr(blk.kv_cache, k).copy_from_numpy(host)
            blk.kv_cache.refresh_shadow()  # a captured frame only converts the rows its own appends write
        self.gen.set_frame_t(snap["frame_t"])
        self._frame = snap["frame"]
        self._rng.bit_generator.state = snap["rng"]
        _stream.synchronize()

    def append_frame(self, latent, ctrl=None):
        """Commit a given latent frame to the KV caches (one NFE at the last sigma, ring writes on) and
        advance the frame counter (``src/quark/engine/cuda.py:177-195`` without the VAE)."""
        self._noise_host.array[:] = self._to_bf16(latent)
        self._h2d(self._append_dev, self._noise_host.ptr, self.cfg.latent_numel * 2)
        ctrl_emb = self.model.encode_ctrl(self._encode_ctrl(ctrl))
        self.model(self._append_dev, sigma_idx=self.gen.n_denoise, frame_t=self.gen.frame_t, ctrl_emb=ctrl_emb, frozen=False)
        from . import functional as qf

        qf.increment(self.gen.frame_t)
        _stream.synchronize()
        self._frame += 1
        return np.asarray(latent)

    def gen_frame(self, ctrl=None, return_img: bool = True, *, noise=None):
        """Generate the next latent frame: 4 denoise NFEs + 1 commit NFE (``engine/cuda.py:197-255``).

        ``noise`` (optional) is a latent-shaped array used instead of the engine's own seeded normal
        noise.  Returns the latent as a bf16-carrier ``uint16`` array ``[1, C, 2H, 2W]`` when
        ``return_img`` is true (there is no VAE to make pixels), else None.
        """
        ctrl_dev = self._encode_ctrl(ctrl)
        n = self.cfg.latent_numel
        if noise is None and self._device_noise:
            from . import functional as qf

            # one draw per frame: frame f uses the Philox counters [f * stride, f * stride + n / 4)
            qf.randn(shape=(1, n), dtype="bf16", counter_offset=self.gen.frame_t, out=self._noise_dev, counter_stride=(n + 3) // 4,
                     seed0=self._noise_seeds[0], seed1=self._noise_seeds[1])  # fmt: skip
        else:
            if noise is None:
                noise = self._rng.standard_normal(n, dtype=np.float32)
            self._noise_host.array[:] = self._to_bf16(noise)
            self._h2d(self._noise_dev, self._noise_host.ptr, n * 2)
        if self._use_graph and self.gen._graph is None:
            self._capture()
        if self._watchdog is not None:  # the guard ends only when the frame has: the host waits for the stream inside it
            with self._watchdog.guard():
                out = self.gen(self._noise_dev, ctrl_dev)
                _stream.synchronize()
        else:
            out = self.gen(self._noise_dev, ctrl_dev)
        self._frame += 1
        if not return_img:
            return None
        self._d2h(self._out_host.ptr, out, n * 2)
        _stream.synchronize()
        return self._out_host.array.reshape(self._latent_shape()).copy()

    def _capture(self) -> None:
        """Capture the frame graph without disturbing the session: the warm-up and capture passes
        write the tail slot and (commit pass) a ring slot of every layer, so snapshot and restore."""
        saved = []
        for blk in self.model.blocks:
            kc = blk.kv_cache
            saved.append([(t, t.to_numpy()) for t in (kc.K_cache, kc.Vt_cache, kc.segments, kc.n_segments)])
        self.gen.prepare_graph(self._noise_dev, self._ctrl_dev, start_frame_t=self._frame)
        for items in saved:
            for t, host in items:
                t.copy_from_numpy(host)
        for blk in self.model.blocks:
            blk.kv_cache.refresh_shadow()
        _stream.synchronize()
