"""Two-phase state restoration shared by modules, optimizers, AMP and checkpoint loading.

Each owner first *prepares* (validates and converts everything without touching live state)
and returns a ``PreparedLoad``; ``commit_prepared`` then publishes the owners in order and, if
one of them raises, rolls back every owner that was attempted, in reverse.
(reference project: python/orthon/_state.py:4-31)
"""


class PreparedLoad:
    __slots__ = ("commit", "rollback", "placement")

    def __init__(self, commit, rollback, placement=None):
        self.commit = commit
        self.rollback = rollback
        self.placement = placement


def commit_prepared(participants):
    done = []
    try:
        for part in participants:
            done.append(part)  # a commit that fails half-way must be rolled back too
            part.commit()
    except BaseException as original:
        problems = []
        for part in reversed(done):
            try:
                part.rollback()
            except BaseException as exc:  # noqa: BLE001
                problems.append(exc)
        if problems:
            raise RuntimeError(
                "checkpoint: transaction rollback failed (%s)" % "; ".join(str(p) for p in problems)
            ) from original
        raise


_PreparedLoad = PreparedLoad
_commit_prepared = commit_prepared
