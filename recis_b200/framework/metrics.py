"""Global metric registry merged into every step's metric dict (``recis/framework/metrics.py:25-38``)."""
GLOBAL_METRICS = {}


def get_global_metrics():
    return GLOBAL_METRICS


def add_metric(name, metric):
    GLOBAL_METRICS[name] = metric
