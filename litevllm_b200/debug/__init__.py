from .activation_sniffer import ActivationSniffer

__all__ = ["ActivationSniffer"]
