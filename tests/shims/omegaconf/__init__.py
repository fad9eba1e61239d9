class DictConfig(dict):
    pass


class OmegaConf:
    @staticmethod
    def to_container(cfg, **kwargs):
        return cfg
