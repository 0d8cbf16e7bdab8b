"
ף<Bx_scale