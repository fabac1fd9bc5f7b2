"""Hook base class: callbacks around training / evaluation / epochs / steps (``recis/hooks/hook.py:1-93``)."""


class Hook:
    def before_train(self): pass
    def after_train(self): pass
    def before_evaluate(self): pass
    def after_evaluate(self): pass
    def before_epoch(self): pass
    def after_epoch(self): pass
    def before_step(self): pass
    def after_step(self, metrics=None, global_step=0): pass
    def end(self): pass
