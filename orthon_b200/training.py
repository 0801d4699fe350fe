"""Supervised-training helpers for classification loops.

`train_step` and `eval_step` return one metrics record per batch: {"loss", "accuracy",
"num_examples"}; `weighted_metric_average` folds such records into the epoch's means, weighting
each batch by its size.  Targets may be a tensor or any sequence of integers.
(reference project: python/orthon/training.py:10-68)"""

_METRICS = ("loss", "accuracy")


def _labels(targets):
    flat = targets.tolist() if hasattr(targets, "tolist") else list(targets)
    return list(map(int, flat))


def classification_accuracy(logits, targets):
    """Share of the rows of [N, C] `logits` whose largest entry sits at the target index."""
    labels = _labels(targets)
    hits = 0
    for guess, label in zip(_labels(logits.argmax(1)), labels):
        hits += guess == label
    return hits / len(labels)


def _forward_metrics(model, inputs, labels, loss_fn):
    logits = model(inputs)
    loss = loss_fn(logits, labels)
    return loss, lambda: {"loss": float(loss.item()), "accuracy": classification_accuracy(logits, labels),
                          "num_examples": len(labels)}


def train_step(model, batch_x, batch_y, loss_fn, optimizer):
    """One optimisation step in training mode; the record describes the batch before the update."""
    labels = _labels(batch_y)
    model.train()
    optimizer.zero_grad()
    loss, record = _forward_metrics(model, batch_x, labels, loss_fn)
    loss.backward()
    optimizer.step()
    return record()


def eval_step(model, batch_x, batch_y, loss_fn):
    """Metrics of one batch in evaluation mode; nothing is updated."""
    model.eval()
    _, record = _forward_metrics(model, batch_x, _labels(batch_y), loss_fn)
    return record()


def weighted_metric_average(step_outputs):
    records = list(step_outputs)
    examples = sum(r["num_examples"] for r in records)
    if examples == 0:
        raise ValueError("weighted_metric_average() requires at least one example")
    summary = {name: sum(r[name] * r["num_examples"] for r in records) / examples for name in _METRICS}
    summary["num_examples"] = examples
    return summary


__all__ = ["classification_accuracy", "train_step", "eval_step", "weighted_metric_average"]
