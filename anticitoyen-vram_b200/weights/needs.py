"""What a model asks of a weight file: tensor names with their shapes and roles."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorNeed:
    """One tensor that a part reads by name.

    ``role`` decides the random initialisation ("matrix", "embedding" and "bias":
    N(0, 0.02); "norm": 1 + N(0, 0.1); "table": integers) and nothing else;
    ``optional`` tensors may be absent from the file (a tied output head).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


class WeightError(ValueError):
    """A weight file that does not fit the model; lists every fault at once."""

    def __init__(self, where: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the configuration asks {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))
