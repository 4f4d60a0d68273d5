"""Layer-weight streaming from host memory (reference: zenyx/streaming/parameter_streamer.py:13-90):
``ParameterStore`` keeps one flat host copy per layer, ``LayerWeightStreamer`` prefetches the next
layer's weights on a side stream while the current layer computes. Unlike the reference, the host
copies are pinned once at registration (not on every fetch) and ``bind`` writes the streamed
weights into the layer's parameters, so the streamed bytes are the ones the layer computes with."""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional

import torch
import torch.nn as nn


class ParameterStore:
    def __init__(self, pin: Optional[bool] = None):
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._flat: Dict[str, torch.Tensor] = {}
        self._layout: Dict[str, List[tuple]] = {}

    def register(self, name: str, module: nn.Module) -> None:
        sd = module.state_dict()
        layout, parts, off = [], [], 0
        for k, v in sd.items():
            n = v.numel()
            layout.append((k, tuple(v.shape), v.dtype, off, n))
            parts.append(v.detach().reshape(-1).to(torch.float32).cpu())
            off += n
        flat = torch.cat(parts) if parts else torch.empty(0)
        self._flat[name] = flat.pin_memory() if (self.pin and flat.numel()) else flat
        self._layout[name] = layout

    def get(self, name: str) -> torch.Tensor:
        return self._flat[name]

    def layout(self, name: str) -> List[tuple]:
        return self._layout[name]

    def names(self) -> List[str]:
        return list(self._flat)

    def nbytes(self, name: str) -> int:
        f = self._flat[name]
        return f.numel() * f.element_size()


class LayerWeightStreamer:
    def __init__(self, store: ParameterStore, device, min_block_bytes: int = 5 << 20, max_resident_layers: int = 2):
        self.store, self.device = store, torch.device(device)
        self.min_block_bytes, self.max_resident_layers = min_block_bytes, max_resident_layers
        self._resident: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self._events: Dict[str, "torch.cuda.Event"] = {}
        self._stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.bytes_streamed = 0

    def prefetch(self, name: str) -> None:
        if name in self._resident:
            return
        host = self.store.get(name)
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                dev = host.to(self.device, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
            self._events[name] = ev
        else:
            dev = host.to(self.device)
        self._resident[name] = dev
        self.bytes_streamed += self.store.nbytes(name)
        while len(self._resident) > self.max_resident_layers:
            old = next(iter(self._resident))
            if old == name:
                break
            self.evict(old)

    def get(self, name: str) -> torch.Tensor:
        if name not in self._resident:
            self.prefetch(name)
        ev = self._events.pop(name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        self._resident.move_to_end(name)
        return self._resident[name]

    def bind(self, name: str, module: nn.Module) -> None:
        """Copies the streamed flat weights into the module's parameters and buffers."""
        flat = self.get(name)
        sd = module.state_dict()
        with torch.no_grad():
            for key, shape, dtype, off, n in self.store.layout(name):
                sd[key].copy_(flat[off: off + n].view(shape).to(dtype))

    def evict(self, name: str) -> None:
        self._resident.pop(name, None)
        self._events.pop(name, None)

    def resident(self) -> List[str]:
        return list(self._resident)
