function [A, info] = psb_bin_read(name)
% PSB_BIN_READ  Load a binary matrix name.{info,offset,index,value} as a MATLAB / Octave matrix.
%   Sparse matrices come back as sparse double (binary ones with all values 1), dense ones as full.
%   Labels written next to a data set are a raw float file: y = psb_array_read([name '.label'], 'single').
% Counterpart of the reference's bin2mat.m (src/data/matlab/bin2mat.m).
  info = psb_bin_info(name);
  vtype = 'single'; if info.sizeof_value == 8, vtype = 'double'; end
  if strcmp(info.type, 'DENSE')
    v = double(psb_array_read([name '.value'], vtype));
    if info.row_major, A = reshape(v, info.cols, info.rows)'; else, A = reshape(v, info.rows, info.cols); end
    return
  end
  itype = 'uint64'; if info.sizeof_index == 4, itype = 'uint32'; end
  off = double(psb_array_read([name '.offset'], 'uint64'));
  idx = double(psb_array_read([name '.index'], itype)) + 1;       % 1-based
  if strcmp(info.type, 'SPARSE_BINARY')
    val = ones(numel(idx), 1);
  else
    val = double(psb_array_read([name '.value'], vtype));
  end
  outer = numel(off) - 1;
  len = diff(off);
  major = repelem((1:outer)', len);                               % outer index of every stored element
  if info.row_major
    A = sparse(major, idx, val, info.rows, info.cols);
  else
    A = sparse(idx, major, val, info.rows, info.cols);
  end
end
