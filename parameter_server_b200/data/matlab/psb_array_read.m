function a = psb_array_read(path, type, first, count)
% PSB_ARRAY_READ  Read a raw little-endian array file (the .offset / .index / .value / .label files).
%   a = psb_array_read(path, type)                 whole file, e.g. type = 'uint64', 'uint32', 'single'
%   a = psb_array_read(path, type, first, count)   count elements starting at element `first` (0-based)
% Counterpart of the reference's load_bin.m (src/data/matlab/load_bin.m).
  if nargin < 3, first = 0; end
  if nargin < 4, count = inf; end
  fid = fopen(path, 'r', 'ieee-le');
  if fid < 0, error('psb:io', 'cannot open %s', path); end
  closer = onCleanup(@() fclose(fid));
  width = numel(typecast(cast(0, type), 'uint8'));
  if first > 0 && fseek(fid, first * width, 'bof') ~= 0
    error('psb:io', '%s is shorter than %d elements', path, first);
  end
  a = fread(fid, count, ['*' type]);
end
