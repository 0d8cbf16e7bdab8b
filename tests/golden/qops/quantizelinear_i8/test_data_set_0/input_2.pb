*
ûÿÿÿÿÿÿÿÿBy_zero_point