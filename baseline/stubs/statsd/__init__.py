"""Stand-in for `statsd`, which this image lacks: a client that drops every metric."""


class StatsClient:
    def __init__(self, *args, **kwargs):
        pass

    def __getattr__(self, name):
        return lambda *args, **kwargs: None
