"""Element-count value that works both as an int and as a call (``t.numel`` / ``t.numel()``)."""


class _Numel(int):
    __slots__ = ()

    def __call__(self):
        return int(self)
