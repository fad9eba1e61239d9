class LightningModule:
    pass


class LightningDataModule:
    pass


class Trainer:
    pass


class Callback:
    pass


from . import loggers, utilities  # noqa: E402,F401
