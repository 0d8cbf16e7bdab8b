"
ף<Ba_scale