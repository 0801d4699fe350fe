"""Small supervised-training helpers (reference project: python/orthon/training.py:10-68)."""


def _as_int_list(targets):
    values = targets.tolist() if hasattr(targets, "tolist") else targets
    return [int(v) for v in values]


def classification_accuracy(logits, targets):
    """Fraction of rows of [N, C] logits whose arg-max equals the integer target."""
    wanted = _as_int_list(targets)
    predicted = _as_int_list(logits.argmax(1))
    return sum(int(p == t) for p, t in zip(predicted, wanted)) / len(wanted)


def train_step(model, batch_x, batch_y, loss_fn, optimizer):
    targets = _as_int_list(batch_y)
    model.train()
    optimizer.zero_grad()
    logits = model(batch_x)
    loss = loss_fn(logits, targets)
    loss.backward()
    optimizer.step()
    return {"loss": float(loss.item()), "accuracy": classification_accuracy(logits, targets), "num_examples": len(targets)}


def eval_step(model, batch_x, batch_y, loss_fn):
    targets = _as_int_list(batch_y)
    model.eval()
    logits = model(batch_x)
    loss = loss_fn(logits, targets)
    return {"loss": float(loss.item()), "accuracy": classification_accuracy(logits, targets), "num_examples": len(targets)}


def weighted_metric_average(step_outputs):
    total = sum(r["num_examples"] for r in step_outputs)
    if total == 0:
        raise ValueError("weighted_metric_average() requires at least one example")
    return {
        "loss": sum(r["loss"] * r["num_examples"] for r in step_outputs) / total,
        "accuracy": sum(r["accuracy"] * r["num_examples"] for r in step_outputs) / total,
        "num_examples": total,
    }
